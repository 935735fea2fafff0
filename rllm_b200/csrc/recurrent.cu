// Recurrent mixers over a per-request state: a short causal convolution with its tail kept between steps, the
// gates of the recurrence, the recurrence itself in two forms, and the gated norm that follows. Float arithmetic
// throughout; the projections that feed it arrive in the run's storage type.
//
// short_conv: y[t, c] = act(b[c] + sum_j w[c, j] * x[t - (taps - 1 - j), c]) over a sequence's own tokens; inputs
//   before the portion come from the slot's tail (the last taps - 1 inputs, oldest first), inputs before position 0
//   are zero. short_conv_keep writes the new tail afterwards (one thread per (sequence, channel) reads the old tail
//   and the portion's last inputs, then writes).
// unit_heads: x <- scale * x / sqrt(sum(x^2) + eps) per (token, head), in place.
// softplus_decay: d = softplus(z + b), a = exp(-exp(A[head]) * d) per column; either is optional as an output.
// state_scan: per head, with key channels k < dim and value columns v < vdim, for each token in order
//     S[k, v] <- a[k] * S[k, v]                      (a per channel, or one per head)
//     u[v]    =  beta * (x[v] - sum_k S[k, v] key[k])    (delta rule)     or   u[v] = f * x[v]   (plain, f optional)
//     S[k, v] <- S[k, v] + key[k] * u[v]
//     o[v]    =  sum_k S[k, v] * query[k]  (+ skip * x[v])
//   A thread owns a value column and every `split`-th key channel (`split` neighbouring lanes share a column and
//   join their sums by shuffles); it keeps its share of S in registers while it walks the sequence's tokens, a few
//   at a time through shared memory. The order of every sum depends on the sizes only, so a position's result is
//   the same bits however its tokens were cut into steps. Queries and keys may be shared by groups of heads.
// gated_norm: per (token, group of columns) y / sqrt(mean(y^2) + eps) * w, with a gate act(g) applied to y before
//   the norm or to the result after it; act silu or sigmoid.
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int MAX_TAPS = 8;

__device__ __forceinline__ void cp_async4(float* smem, const float* gmem, bool pred) {      // pred false: zero
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem);
  const int sz = pred ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_0() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// A CTA a token (blockIdx.x) and 256 channels (blockIdx.y): what a token has of its own is read once a thread.
template <typename TI>
__global__ void short_conv_kernel(const TI* __restrict__ x, long long ld, int col0, int C, int taps,
                                  const float* __restrict__ w, const float* __restrict__ bias,
                                  const int* __restrict__ token_seq, const int* __restrict__ positions,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                  const float* __restrict__ tail, float* __restrict__ out, int silu) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s = token_seq[t], row0 = cu_q[s], pos = positions[t];
  const int slot = state_slots ? state_slots[s] : -1;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;
    if (pos - back < 0) continue;
    const int r = t - back;
    float v = 0.f;
    if (r >= row0) v = to_f32(x[(long long)r * ld + col0 + c]);
    else if (slot >= 0) v = tail[((long long)slot * (taps - 1) + (taps - 1 - (row0 - r))) * C + c];
    acc = fmaf(w[(long long)c * taps + j], v, acc);
  }
  out[(long long)t * C + c] = silu ? acc / (1.f + expf(-acc)) : acc;
}

template <typename TI>
__global__ void short_conv_keep_kernel(const TI* __restrict__ x, long long ld, int col0, int C, int taps,
                                       const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                       float* __restrict__ tail, int S) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)S * C) return;
  const int s = (int)(i / C), c = (int)(i % C);
  const int slot = state_slots[s];
  if (slot < 0) return;
  const int row0 = cu_q[s], n = cu_q[s + 1] - row0, keep = taps - 1;
  float* tp = tail + (long long)slot * keep * C + c;
  float old[MAX_TAPS];
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) old[k] = k < keep ? tp[(long long)k * C] : 0.f;
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) {
    if (k >= keep) break;
    const int at = n + k;                       // index in [old tail | the portion's inputs]
    tp[(long long)k * C] = at < keep ? old[at] : to_f32(x[(long long)(row0 + at - keep) * ld + col0 + c]);
  }
}

__global__ void unit_heads_kernel(float* __restrict__ x, long long ld, int col0, int heads, int dim, float scale, float eps,
                                  int T) {
  pdl_launch();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T * heads) return;
  float* p = x + (long long)(warp / heads) * ld + col0 + (warp % heads) * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) ss = fmaf(p[i], p[i], ss);
  ss = warp_sum(ss);
  const float r = scale / sqrtf(ss + eps);
  for (int i = lane; i < dim; i += 32) p[i] *= r;
}

template <typename TI>
__global__ void softplus_decay_kernel(const TI* __restrict__ z, long long ld, int col0, const float* __restrict__ bias,
                                      const float* __restrict__ a_log, int n, int per_head, float* __restrict__ step,
                                      float* __restrict__ decay, long long total) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / n;
    const int c = (int)(i % n);
    const float d = softplus_f(to_f32(z[t * ld + col0 + c]) + (bias ? bias[c] : 0.f));
    if (step) step[i] = d;
    if (decay) decay[i] = expf(-expf(a_log[c / per_head]) * d);
  }
}

struct ScanArgs {
  const float* q; long long q_ld; int q_heads;        // [T, q_heads * dim] at q (column offset folded in)
  const float* k; long long k_ld; int k_heads;
  const float* v; long long v_ld;                     // [T, H * vdim]
  const float* decay; int decay_per_channel;          // [T, H * dim] or [T, H]
  const void* beta; long long beta_ld;                // logits [T, H] of the projection's type, or null: plain form
  const float* vscale;                                // [T, H] or null
  const float* skip;                                  // [H] or null
  int H, dim, vdim, split, ch, beta_bf16;
  const int* cu_q; const int* state_slots;
  float* state;                                       // [slots, H, dim, vdim]
  float* out;                                         // [T, H, vdim]
};

template <typename TB, int R>
__global__ void __launch_bounds__(128) state_scan_kernel(ScanArgs a) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int dim = a.dim, vdim = a.vdim, split = a.split, ch = a.ch, H = a.H;
  const int cols = 128 / split;                      // value columns of a CTA
  float* qs = sm;                                    // [ch][dim]
  float* ks = qs + ch * dim;
  float* as = ks + ch * dim;                         // [ch][dim] or [ch]
  float* vs = as + (a.decay_per_channel ? ch * dim : ch);   // [ch][cols]
  float* bs = vs + ch * cols;                        // [ch] beta, [ch] vscale
  const int seq = blockIdx.x, h = blockIdx.y;
  const int sub = threadIdx.x % split, col = threadIdx.x / split;
  const int v = blockIdx.z * cols + col;
  const bool vok = v < vdim;
  const int row0 = a.cu_q[seq], row1 = a.cu_q[seq + 1];
  const int slot = a.state_slots ? a.state_slots[seq] : -1;
  const int qh = h / (H / a.q_heads), kh = h / (H / a.k_heads);
  float S[R];
  float* sp = a.state + (((long long)(slot < 0 ? 0 : slot) * H + h) * dim) * vdim + v;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int k = i * split + sub;
    S[i] = (slot >= 0 && vok && k < dim) ? sp[(long long)k * vdim] : 0.f;
  }
  const float skip = a.skip ? a.skip[h] : 0.f;
  const bool delta = a.beta != nullptr;
  for (int c0 = row0; c0 < row1; c0 += ch) {
    const int n = min(ch, row1 - c0);
    __syncthreads();
    for (int x = threadIdx.x; x < n * dim; x += 128) {
      const int cc = x / dim, k = x % dim;
      const long long r = c0 + cc;
      qs[cc * dim + k] = a.q[r * a.q_ld + qh * dim + k];
      ks[cc * dim + k] = a.k[r * a.k_ld + kh * dim + k];
      if (a.decay_per_channel) as[cc * dim + k] = a.decay[(r * H + h) * dim + k];
    }
    for (int x = threadIdx.x; x < n * cols; x += 128) {
      const int cc = x / cols, c = x % cols;
      const int vv = blockIdx.z * cols + c;
      vs[x] = vv < vdim ? a.v[(long long)(c0 + cc) * a.v_ld + h * vdim + vv] : 0.f;
    }
    for (int cc = threadIdx.x; cc < n; cc += 128) {
      const long long r = c0 + cc;
      if (!a.decay_per_channel) as[cc] = a.decay[r * H + h];
      bs[cc] = delta ? sigmoid_f(to_f32(reinterpret_cast<const TB*>(a.beta)[r * a.beta_ld + h])) : 1.f;
      bs[ch + cc] = a.vscale ? a.vscale[r * H + h] : 1.f;
    }
    __syncthreads();
    for (int cc = 0; cc < n; ++cc) {
      const float* kr = ks + cc * dim;
      const float* qr = qs + cc * dim;
      const float x = vs[cc * cols + col];
      float u;
      if (a.decay_per_channel) {
        const float* ar = as + cc * dim;
#pragma unroll
        for (int i = 0; i < R; ++i) { const int k = i * split + sub; if (k < dim) S[i] *= ar[k]; }
      } else {
        const float al = as[cc];
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] *= al;
      }
      if (delta) {
        float r = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) { const int k = i * split + sub; if (k < dim) r = fmaf(S[i], kr[k], r); }
        for (int o = 1; o < split; o <<= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        u = bs[cc] * (x - r);
      } else {
        u = bs[ch + cc] * x;
      }
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int k = i * split + sub;
        if (k < dim) { S[i] = fmaf(kr[k], u, S[i]); o = fmaf(S[i], qr[k], o); }
      }
      for (int w = 1; w < split; w <<= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
      if (sub == 0 && vok) a.out[((long long)(c0 + cc) * H + h) * vdim + v] = fmaf(skip, x, o);
    }
  }
  if (slot >= 0 && vok) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int k = i * split + sub;
      if (k < dim) sp[(long long)k * vdim] = S[i];
    }
  }
}

// One CTA per (token, group). gate: logits [T, >= cols] with row stride g_ld, of type TG.
template <typename TG, typename TO>
__global__ void gated_norm_kernel(const float* __restrict__ y, const TG* __restrict__ gate, long long g_ld,
                                  const float* __restrict__ w, int w_period, float eps, TO* __restrict__ out, int groups,
                                  int gsize, int gate_first, int act) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const long long t = blockIdx.x / groups;
  const int g = blockIdx.x % groups;
  const int n = groups * gsize;
  const float* yr = y + t * n + (long long)g * gsize;
  const TG* gr = gate ? gate + t * g_ld + (long long)g * gsize : nullptr;
  auto gv = [&](int i) {
    if (!gr) return 1.f;
    const float z = to_f32(gr[i]);
    return act == 0 ? z / (1.f + expf(-z)) : 1.f / (1.f + expf(-z));
  };
  float ss = 0.f;
  for (int i = threadIdx.x; i < gsize; i += blockDim.x) {
    const float v = gate_first ? yr[i] * gv(i) : yr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)gsize + eps);
  TO* o = out + t * n + (long long)g * gsize;
  for (int i = threadIdx.x; i < gsize; i += blockDim.x) {
    const float wi = w[(g * gsize + i) % w_period];
    const float v = gate_first ? yr[i] * gv(i) * r * wi : yr[i] * r * wi * gv(i);
    o[i] = from_f32<TO>(v);
  }
}

inline unsigned blocks_for(long long n) { return (unsigned)((n + 255) / 256 > 65535 * 8 ? 65535 * 8 : (n + 255) / 256); }

// The same recurrence for heads of R * SPLIT key channels (32 to 256) with R = 32, 16 or 8 channels a thread, the sizes
// known when compiled: a thread's channels are neighbours (sub * R ...), so queries, keys and decays come from shared
// memory in pieces of four (rows padded by four floats a lane share, which keeps the shares on different banks),
// and the sums over channels run as four chains side by side. Fewer channels a thread means fewer value columns a
// CTA and more CTAs a head; R depends on the sizes alone, so a position's result is the same bits whatever the cut
// into steps and whatever else is in the batch.
template <int R, int SPLIT, bool PERCH>
__global__ void __launch_bounds__(128) state_scan_fast_kernel(ScanArgs a) {
  pdl_launch();
  pdl_wait();
  constexpr int DIM = R * SPLIT, LDK = SPLIT * (R + 4), COLS = 128 / SPLIT;
  extern __shared__ __align__(16) float sm[];
  const int vdim = a.vdim, ch = a.ch, H = a.H;
  // a stage: queries [ch][LDK], keys [ch][LDK], decays [ch][LDK] or [ch], values [ch][COLS], beta [ch], vscale [ch]
  const int stg = (ch * LDK * (PERCH ? 3 : 2) + (PERCH ? 0 : ch) + ch * COLS + 2 * ch + 3) & ~3;
  const int seq = blockIdx.x, h = blockIdx.y;
  const int sub = threadIdx.x % SPLIT, col = threadIdx.x / SPLIT;
  const int v = blockIdx.z * COLS + col;
  const bool vok = v < vdim;
  const int row0 = a.cu_q[seq], row1 = a.cu_q[seq + 1];
  const int slot = a.state_slots ? a.state_slots[seq] : -1;
  const int qh = h / (H / a.q_heads), kh = h / (H / a.k_heads);
  float S[R];
  float* sp = a.state + (((long long)(slot < 0 ? 0 : slot) * H + h) * DIM + sub * R) * vdim + v;
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = (slot >= 0 && vok) ? sp[(long long)i * vdim] : 0.f;
  const float skip = a.skip ? a.skip[h] : 0.f;
  const bool delta = a.beta != nullptr;
  // The next tokens' rows travel into the other stage (cp.async, four bytes a copy: the columns of a view need no
  // alignment) while this stage's tokens are worked on; the few numbers a token has per head (decay, beta, value
  // scale) wait in registers of the first threads meanwhile.
  auto issue = [&](int c0, int stage) {
    float* qs = sm + stage * stg;
    float* ks = qs + ch * LDK;
    float* as = ks + ch * LDK;
    float* vs = as + (PERCH ? ch * LDK : ch);
    const int n = min(ch, row1 - c0);
    for (int x = threadIdx.x; x < n * DIM; x += 128) {
      const int cc = x / DIM, k = x % DIM;
      const long long r = c0 + cc;
      const int at = cc * LDK + (k / R) * (R + 4) + k % R;
      cp_async4(qs + at, a.q + r * a.q_ld + qh * DIM + k, true);
      cp_async4(ks + at, a.k + r * a.k_ld + kh * DIM + k, true);
      if (PERCH) cp_async4(as + at, a.decay + (r * H + h) * DIM + k, true);
    }
    for (int x = threadIdx.x; x < n * COLS; x += 128) {
      const int cc = x / COLS, vv = blockIdx.z * COLS + x % COLS;
      cp_async4(vs + x, a.v + (long long)(c0 + cc) * a.v_ld + h * vdim + (vv < vdim ? vv : 0), vv < vdim);
    }
  };
  float n_al = 1.f, n_b = 0.f, n_vs = 1.f;
  auto few_load = [&](int c0) {
    if ((int)threadIdx.x < min(ch, row1 - c0)) {
      const long long r = c0 + threadIdx.x;
      if (!PERCH) n_al = a.decay[r * H + h];
      if (delta) n_b = a.beta_bf16 ? to_f32(reinterpret_cast<const bf16*>(a.beta)[r * a.beta_ld + h])
                                   : reinterpret_cast<const float*>(a.beta)[r * a.beta_ld + h];
      if (a.vscale) n_vs = a.vscale[r * H + h];
    }
  };
  auto few_store = [&](int stage) {
    if ((int)threadIdx.x < ch) {
      float* as = sm + stage * stg + 2 * ch * LDK;
      float* bs = as + (PERCH ? ch * LDK : ch) + ch * COLS;
      if (!PERCH) as[threadIdx.x] = n_al;
      bs[threadIdx.x] = delta ? sigmoid_f(n_b) : 1.f;
      bs[ch + threadIdx.x] = n_vs;
    }
  };
  const int chunks = (row1 - row0 + ch - 1) / ch;
  if (chunks > 0) {
    issue(row0, 0);
    few_load(row0);
    few_store(0);
  }
  cp_async_commit();
  for (int ci = 0; ci < chunks; ++ci) {
    const int c0 = row0 + ci * ch, stage = ci & 1;
    const int n = min(ch, row1 - c0);
    if (ci + 1 < chunks) {
      issue(c0 + ch, stage ^ 1);
      few_load(c0 + ch);
    }
    cp_async_commit();
    cp_async_wait_1();
    __syncthreads();
    const float* qs = sm + stage * stg;
    const float* ks = qs + ch * LDK;
    const float* as = ks + ch * LDK;
    const float* vs = as + (PERCH ? ch * LDK : ch);
    const float* bs = vs + ch * COLS;
    for (int cc = 0; cc < n; ++cc) {
      const float4* kr = reinterpret_cast<const float4*>(ks + cc * LDK + sub * (R + 4));
      const float4* qr = reinterpret_cast<const float4*>(qs + cc * LDK + sub * (R + 4));
      const float x = vs[cc * COLS + col];
      float kk[R];
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 t = kr[i];
        kk[4 * i] = t.x; kk[4 * i + 1] = t.y; kk[4 * i + 2] = t.z; kk[4 * i + 3] = t.w;
      }
      if (PERCH) {
        const float4* ar = reinterpret_cast<const float4*>(as + cc * LDK + sub * (R + 4));
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          const float4 t = ar[i];
          S[4 * i] *= t.x; S[4 * i + 1] *= t.y; S[4 * i + 2] *= t.z; S[4 * i + 3] *= t.w;
        }
      } else {
        const float al = as[cc];
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] *= al;
      }
      float u;
      if (delta) {
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          r0 = fmaf(S[i], kk[i], r0); r1 = fmaf(S[i + 1], kk[i + 1], r1);
          r2 = fmaf(S[i + 2], kk[i + 2], r2); r3 = fmaf(S[i + 3], kk[i + 3], r3);
        }
        float r = (r0 + r1) + (r2 + r3);
#pragma unroll
        for (int o = 1; o < SPLIT; o <<= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        u = bs[cc] * (x - r);
      } else {
        u = bs[ch + cc] * x;
      }
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 t = qr[i];
        S[4 * i] = fmaf(kk[4 * i], u, S[4 * i]); o0 = fmaf(S[4 * i], t.x, o0);
        S[4 * i + 1] = fmaf(kk[4 * i + 1], u, S[4 * i + 1]); o1 = fmaf(S[4 * i + 1], t.y, o1);
        S[4 * i + 2] = fmaf(kk[4 * i + 2], u, S[4 * i + 2]); o2 = fmaf(S[4 * i + 2], t.z, o2);
        S[4 * i + 3] = fmaf(kk[4 * i + 3], u, S[4 * i + 3]); o3 = fmaf(S[4 * i + 3], t.w, o3);
      }
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int w = 1; w < SPLIT; w <<= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
      if (sub == 0 && vok) a.out[((long long)(c0 + cc) * H + h) * vdim + v] = fmaf(skip, x, o);
    }
    if (ci + 1 < chunks) few_store(stage ^ 1);
    __syncthreads();            // this stage is free for the copy after the next
  }
  cp_async_wait_0();
  if (slot >= 0 && vok) {
#pragma unroll
    for (int i = 0; i < R; ++i) sp[(long long)i * vdim] = S[i];
  }
}

int launch_scan_fast(const ScanArgs& a, int r, bool perch, dim3 grid, size_t smem, cudaStream_t s) {
#define RLLM_SF(RR, SP)                                                                                            \
  if (r == RR && a.split == SP)                                                                                    \
    return perch ? launch_ex(state_scan_fast_kernel<RR, SP, true>, grid, dim3(128), smem, s, 1, a)                 \
                 : launch_ex(state_scan_fast_kernel<RR, SP, false>, grid, dim3(128), smem, s, 1, a)
  RLLM_SF(32, 1); RLLM_SF(32, 2); RLLM_SF(32, 4); RLLM_SF(32, 8);
  RLLM_SF(16, 2); RLLM_SF(16, 4); RLLM_SF(16, 8); RLLM_SF(16, 16);
  RLLM_SF(8, 4); RLLM_SF(8, 8); RLLM_SF(8, 16); RLLM_SF(8, 32);
#undef RLLM_SF
  return ERR_BAD_SIZE;
}

}  // namespace

RLLM_API int rllm_short_conv(int dt, const void* x, long long ld, int col0, int C, int taps, const float* w, const float* bias,
                             const int* token_seq, const int* positions, const int* cu_q, const int* state_slots,
                             float* tail, float* out, int T, int S, int silu, void* stream) {
  if (T <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS) return ERR_BAD_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = C >= 256 ? 256 : C >= 128 ? 128 : 64;
  const dim3 grid((unsigned)T, (unsigned)((C + threads - 1) / threads));
  if (grid.y > 65535) return ERR_TOO_LARGE;
  int rc;
  if (dt == DT_F32)
    rc = launch_ex(short_conv_kernel<float>, grid, dim3(threads), 0, s, 1, (const float*)x, ld, col0, C, taps, w, bias,
                   token_seq, positions, cu_q, state_slots, (const float*)tail, out, silu);
  else if (dt == DT_BF16)
    rc = launch_ex(short_conv_kernel<bf16>, grid, dim3(threads), 0, s, 1, (const bf16*)x, ld, col0, C, taps, w, bias,
                   token_seq, positions, cu_q, state_slots, (const float*)tail, out, silu);
  else return ERR_BAD_DTYPE;
  if (rc || taps == 1 || state_slots == nullptr || tail == nullptr) return rc;
  const unsigned blocks = (unsigned)(((long long)S * C + 255) / 256);
  if (dt == DT_F32)
    return launch_ex(short_conv_keep_kernel<float>, dim3(blocks), dim3(256), 0, s, 1, (const float*)x, ld, col0, C, taps, cu_q,
                     state_slots, tail, S);
  return launch_ex(short_conv_keep_kernel<bf16>, dim3(blocks), dim3(256), 0, s, 1, (const bf16*)x, ld, col0, C, taps, cu_q,
                   state_slots, tail, S);
}

RLLM_API int rllm_unit_heads(float* x, long long ld, int col0, int heads, int dim, float scale, float eps, int T, void* stream) {
  if (T <= 0 || heads <= 0) return 0;
  const long long warps = (long long)T * heads;
  return launch_ex(unit_heads_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, 1, x, ld, col0, heads,
                   dim, scale, eps, T);
}

RLLM_API int rllm_softplus_decay(int dt, const void* z, long long ld, int col0, const float* bias, const float* a_log, int T,
                                 int n, int per_head, float* step, float* decay, void* stream) {
  if (T <= 0 || n <= 0) return 0;
  if (per_head <= 0 || n % per_head) return ERR_BAD_SIZE;
  const long long total = (long long)T * n;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32)
    return launch_ex(softplus_decay_kernel<float>, dim3(blocks_for(total)), dim3(256), 0, s, 1, (const float*)z, ld, col0, bias,
                     a_log, n, per_head, step, decay, total);
  if (dt == DT_BF16)
    return launch_ex(softplus_decay_kernel<bf16>, dim3(blocks_for(total)), dim3(256), 0, s, 1, (const bf16*)z, ld, col0, bias,
                     a_log, n, per_head, step, decay, total);
  return ERR_BAD_DTYPE;
}

// How the key channels of a head are dealt to lanes: `split` neighbouring lanes share a value column.
RLLM_API int rllm_state_scan_split(int dim) {
  int split = 1;
  while (32 * split < dim && split < 32) split <<= 1;
  return split;
}

// Channels a thread for the kernel with compiled sizes (0: the general kernel). 32 measured best for single tokens at
// every batch (fewer channels a thread mean more CTAs that each stage a head's whole queries and keys) and within a
// tenth of the best for one long prompt; `want` (16 or 8) asks for fewer, for measurements.
static int scan_fast_channels(int dim, int want) {
  if (dim != 32 && dim != 64 && dim != 128 && dim != 256) return 0;
  int r = (want == 16 || want == 8) ? want : 32;
  while (dim / r > 32) r <<= 1;
  return r;
}

RLLM_API int rllm_state_scan(int beta_dt, const float* q, long long q_ld, int q_heads, const float* k, long long k_ld,
                             int k_heads, const float* v, long long v_ld, const float* decay, int decay_per_channel,
                             const void* beta, long long beta_ld, const float* vscale, const float* skip, int S, int H,
                             int dim, int vdim, const int* cu_q, const int* state_slots, float* state, float* out,
                             int channels, void* stream) {
  if (S <= 0) return 0;
  if (H <= 0 || dim <= 0 || dim > 1024 || vdim <= 0 || q_heads <= 0 || k_heads <= 0 || H % q_heads || H % k_heads)
    return ERR_BAD_SIZE;
  ScanArgs a;
  a.q = q; a.q_ld = q_ld; a.q_heads = q_heads; a.k = k; a.k_ld = k_ld; a.k_heads = k_heads; a.v = v; a.v_ld = v_ld;
  a.decay = decay; a.decay_per_channel = decay_per_channel; a.beta = beta; a.beta_ld = beta_ld; a.vscale = vscale;
  a.skip = skip; a.H = H; a.dim = dim; a.vdim = vdim; a.cu_q = cu_q; a.state_slots = state_slots; a.state = state; a.out = out;
  a.split = rllm_state_scan_split(dim);
  a.ch = dim <= 128 ? 16 : dim <= 256 ? 8 : dim <= 512 ? 4 : 2;
  a.beta_bf16 = beta != nullptr && beta_dt == DT_BF16;
  if (beta != nullptr && beta_dt != DT_BF16 && beta_dt != DT_F32) return ERR_BAD_DTYPE;
  cudaStream_t s = (cudaStream_t)stream;
  if (const int r = scan_fast_channels(dim, channels)) {
    a.split = dim / r;
    const int fcols = 128 / a.split, ldk = a.split * (r + 4);
    a.ch = a.ch > 2 ? a.ch / 2 : 1;                  // two stages in the room of one
    const size_t stage = ((size_t)a.ch * ldk * (decay_per_channel ? 3 : 2) + (decay_per_channel ? 0 : a.ch) +
                          (size_t)a.ch * fcols + 2 * a.ch + 3) & ~(size_t)3;
    const size_t fsmem = sizeof(float) * 2 * stage;
    return launch_scan_fast(a, r, decay_per_channel != 0, dim3(S, H, (vdim + fcols - 1) / fcols), fsmem, s);
  }
  const int cols = 128 / a.split;
  const size_t smem = sizeof(float) * ((size_t)a.ch * dim * (decay_per_channel ? 3 : 2) + (decay_per_channel ? 0 : a.ch) +
                                       (size_t)a.ch * cols + 2 * a.ch);
  const dim3 grid(S, H, (vdim + cols - 1) / cols);
  const bool small = dim <= 16;
  if (beta == nullptr || beta_dt == DT_F32)
    return small ? launch_ex(state_scan_kernel<float, 16>, grid, dim3(128), smem, s, 1, a)
                 : launch_ex(state_scan_kernel<float, 32>, grid, dim3(128), smem, s, 1, a);
  if (beta_dt == DT_BF16)
    return small ? launch_ex(state_scan_kernel<bf16, 16>, grid, dim3(128), smem, s, 1, a)
                 : launch_ex(state_scan_kernel<bf16, 32>, grid, dim3(128), smem, s, 1, a);
  return ERR_BAD_DTYPE;
}

RLLM_API int rllm_gated_norm(const float* y, const void* gate, int gate_dt, long long g_ld, const float* w, int w_period,
                             float eps, void* out, int out_dt, int T, int groups, int gsize, int gate_first, int act,
                             void* stream) {
  if (T <= 0) return 0;
  if (groups <= 0 || gsize <= 0 || w_period <= 0 || act < 0 || act > 1) return ERR_BAD_SIZE;
  const dim3 grid((unsigned)((long long)T * groups)), block(gsize >= 512 ? 256 : gsize >= 128 ? 128 : 64);
  cudaStream_t s = (cudaStream_t)stream;
#define RLLM_GN(TG, TO) \
  return launch_ex(gated_norm_kernel<TG, TO>, grid, block, 0, s, 1, y, (const TG*)gate, g_ld, w, w_period, eps, (TO*)out, groups, \
                   gsize, gate_first, act)
  if (gate_dt == DT_F32 && out_dt == DT_F32) RLLM_GN(float, float);
  if (gate_dt == DT_F32 && out_dt == DT_BF16) RLLM_GN(float, bf16);
  if (gate_dt == DT_BF16 && out_dt == DT_BF16) RLLM_GN(bf16, bf16);
  if (gate_dt == DT_BF16 && out_dt == DT_F32) RLLM_GN(bf16, float);
#undef RLLM_GN
  return ERR_BAD_DTYPE;
}
