// Grouped-query attention whose heads' softmax weights are mixed by a matrix before they meet the values
// ("talking heads" after the softmax), over the paged cache, with a causal window and an optional sink.
//
//   s_g(i, j) = scale * q_g(i) . k_c(g)(j)                       for the keys j the mask lets position i see
//   p_g(i, j) = exp(s_g(i, j)) / (exp(sink_g) + sum_j' exp(s_g(i, j')))      (no sink: the plain softmax)
//   w_h(i, j) = sum_g M[h, g] p_g(i, j)
//   o_h(i)    = sum_j w_h(i, j) v_c(h)(j)                        c(h): the key/value head of query head h
//
// The mix needs every head's *normalised* weight of a (query, key) pair at once, so a query's keys are walked
// twice: a first pass finds each head's maximum and denominator, a second one recomputes the scores, normalises,
// mixes a tile of 32 keys in shared memory and adds the tile's values. Scores, softmax, mix and sums are float.
//
// talk_attention_simt: one CTA per query token, float arithmetic on the CUDA cores (the 32-bit run, and every size).
//   Warp w owns the heads g with g % warps == w: their running maxima and sums in the first pass, their output
//   columns (lane d, d + 32, ...) in the second. Keys and values of one kv head at a time pass through shared memory.
// talk_attention_mma (talk_attention_mma.cuh): bfloat16 on the tensor cores, one pass, the mix after the values.
// value_norm_store: keys as they are, values divided by their root mean square per head (no weight), into the pages.
#include "common.cuh"
using namespace rllm;
#include "talk_attention_mma.cuh"

namespace {

constexpr int TK = 32;          // keys a tile
constexpr int MAX_HPW = 8;      // heads a warp owns at most
constexpr int MAX_VPL = 8;      // value columns a lane owns at most (vd <= 256)

template <typename T>
__global__ void value_norm_store_kernel(const T* __restrict__ proj, long long ld, int k_off, int v_off, int nkv, int kd,
                                        int vd, float eps, int norm, const int* __restrict__ slots, T* __restrict__ kcache,
                                        T* __restrict__ vcache, int page_size, int Tn) {
  pdl_launch();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= Tn * nkv) return;
  const int t = warp / nkv, c = warp % nkv;
  const int slot = slots[t];
  if (slot < 0) return;
  const int page = slot / page_size, off = slot % page_size;
  const T* kr = proj + (long long)t * ld + k_off + c * kd;
  const T* vr = proj + (long long)t * ld + v_off + c * vd;
  T* kc = kcache + (((long long)page * nkv + c) * page_size + off) * kd;
  T* vc = vcache + (((long long)page * nkv + c) * page_size + off) * vd;
  for (int i = lane; i < kd; i += 32) kc[i] = kr[i];
  float r = 1.f;
  if (norm) {
    float ss = 0.f;
    for (int i = lane; i < vd; i += 32) { const float v = to_f32(vr[i]); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    r = 1.f / sqrtf(ss / (float)vd + eps);
  }
  for (int i = lane; i < vd; i += 32) vc[i] = norm ? from_f32<T>(to_f32(vr[i]) * r) : vr[i];
}

struct TalkArgs {
  const void* q; long long q_ld;
  const void* kcache; const void* vcache;
  const int* token_seq; const int* positions; const int* block_table; long long bt_ld;
  const float* mix;           // [H, H]
  const float* sinks;         // [H] or null
  void* out;                  // [T, H * vd]
  int H, G, kd, vd, page_size, window, chunk, warps;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(512) talk_attention_simt_kernel(TalkArgs a) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int H = a.H, G = a.G, kd = a.kd, vd = a.vd, ps = a.page_size, nw = a.warps;
  const int rep = H / G, kdp = kd + 1;
  float* Q = sm;                               // [H][kd], scaled
  float* KV = Q + H * kd;                      // keys [TK][kd + 1] or values [TK][vd]
  float* P = KV + TK * (kdp > vd ? kdp : vd);  // [H][TK]
  float* Wm = P + H * TK;                      // [H][TK]
  float* M = Wm + H * TK;                      // [H][H]
  float* stat = M + H * H;                     // [H] maximum, [H] 1 / denominator
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = a.token_seq[t], pos = a.positions[t];
  int first = 0;
  if (a.window > 0) first = max(first, pos - a.window + 1);
  if (a.chunk > 0) first = max(first, pos / a.chunk * a.chunk);
  const int* table = a.block_table + (long long)seq * a.bt_ld;
  const T* q = reinterpret_cast<const T*>(a.q) + (long long)t * a.q_ld;
  const T* kc = reinterpret_cast<const T*>(a.kcache);
  const T* vc = reinterpret_cast<const T*>(a.vcache);
  for (int i = threadIdx.x; i < H * kd; i += blockDim.x) Q[i] = to_f32(q[i]) * a.scale;
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) M[i] = a.mix[i];
  const int first_tile = first / TK * TK;

  // ---- pass 1: every head's maximum and sum of exponentials
  float m_run[MAX_HPW], l_run[MAX_HPW];
#pragma unroll
  for (int i = 0; i < MAX_HPW; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }
  for (int j0 = first_tile; j0 <= pos; j0 += TK) {
    for (int c = 0; c < G; ++c) {
      __syncthreads();
      for (int x = threadIdx.x; x < TK * kd; x += blockDim.x) {
        const int jj = x / kd, d = x % kd, j = j0 + jj;
        float v = 0.f;
        if (j >= first && j <= pos) {
          const int page = table[j / ps];
          if (page >= 0) v = to_f32(kc[(((long long)page * G + c) * ps + j % ps) * kd + d]);
        }
        KV[jj * kdp + d] = v;
      }
      __syncthreads();
      const int j = j0 + lane;
      const bool ok = j >= first && j <= pos;
#pragma unroll
      for (int i = 0; i < MAX_HPW; ++i) {
        const int g = warp + i * nw;
        if (g >= H || g / rep != c) continue;
        const float* qg = Q + g * kd;
        const float* kr = KV + lane * kdp;
        float s = 0.f;
        for (int d = 0; d < kd; ++d) s = fmaf(qg[d], kr[d], s);
        if (ok) {
          const float mn = fmaxf(m_run[i], s);
          l_run[i] = l_run[i] * expf(m_run[i] - mn) + expf(s - mn);
          m_run[i] = mn;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_HPW; ++i) {
    const int g = warp + i * nw;
    if (g >= H) continue;
    float m = warp_max(m_run[i]);
    if (a.sinks) m = fmaxf(m, a.sinks[g]);
    float l = l_run[i] > 0.f ? l_run[i] * expf(m_run[i] - m) : 0.f;
    l = warp_sum(l);
    if (a.sinks) l += expf(a.sinks[g] - m);
    if (lane == 0) { stat[g] = m; stat[H + g] = 1.f / l; }
  }

  // ---- pass 2: normalised weights, mixed across heads, times the values
  float acc[MAX_HPW][MAX_VPL];
#pragma unroll
  for (int i = 0; i < MAX_HPW; ++i)
#pragma unroll
    for (int e = 0; e < MAX_VPL; ++e) acc[i][e] = 0.f;
  for (int j0 = first_tile; j0 <= pos; j0 += TK) {
    for (int c = 0; c < G; ++c) {
      __syncthreads();
      for (int x = threadIdx.x; x < TK * kd; x += blockDim.x) {
        const int jj = x / kd, d = x % kd, j = j0 + jj;
        float v = 0.f;
        if (j >= first && j <= pos) {
          const int page = table[j / ps];
          if (page >= 0) v = to_f32(kc[(((long long)page * G + c) * ps + j % ps) * kd + d]);
        }
        KV[jj * kdp + d] = v;
      }
      __syncthreads();
      const int j = j0 + lane;
      const bool ok = j >= first && j <= pos;
#pragma unroll
      for (int i = 0; i < MAX_HPW; ++i) {
        const int g = warp + i * nw;
        if (g >= H || g / rep != c) continue;
        const float* qg = Q + g * kd;
        const float* kr = KV + lane * kdp;
        float s = 0.f;
        for (int d = 0; d < kd; ++d) s = fmaf(qg[d], kr[d], s);
        P[g * TK + lane] = ok ? expf(s - stat[g]) * stat[H + g] : 0.f;
      }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < H * TK; x += blockDim.x) {
      const int h = x / TK, jj = x % TK;
      float w = 0.f;
      for (int g = 0; g < H; ++g) w = fmaf(M[h * H + g], P[g * TK + jj], w);
      Wm[x] = w;
    }
    for (int c = 0; c < G; ++c) {
      __syncthreads();
      for (int x = threadIdx.x; x < TK * vd; x += blockDim.x) {
        const int jj = x / vd, d = x % vd, j = j0 + jj;
        float v = 0.f;
        if (j >= first && j <= pos) {
          const int page = table[j / ps];
          if (page >= 0) v = to_f32(vc[(((long long)page * G + c) * ps + j % ps) * vd + d]);
        }
        KV[jj * vd + d] = v;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < MAX_HPW; ++i) {
        const int h = warp + i * nw;
        if (h >= H || h / rep != c) continue;
        const float* wr = Wm + h * TK;
        for (int jj = 0; jj < TK; ++jj) {
          const float w = wr[jj];
#pragma unroll
          for (int e = 0; e < MAX_VPL; ++e) {
            const int d = lane + 32 * e;
            if (d < vd) acc[i][e] = fmaf(w, KV[jj * vd + d], acc[i][e]);
          }
        }
      }
    }
  }
  T* o = reinterpret_cast<T*>(a.out) + (long long)t * H * vd;
#pragma unroll
  for (int i = 0; i < MAX_HPW; ++i) {
    const int h = warp + i * nw;
    if (h >= H) continue;
#pragma unroll
    for (int e = 0; e < MAX_VPL; ++e) {
      const int d = lane + 32 * e;
      if (d < vd) o[h * vd + d] = from_f32<T>(acc[i][e]);
    }
  }
}

}  // namespace

RLLM_API int rllm_value_norm_store(int dt, const void* proj, long long ld, int k_off, int v_off, int T, int nkv, int kd, int vd,
                                   float eps, int norm, const int* slots, void* kcache, void* vcache, int page_size,
                                   void* stream) {
  if (T <= 0 || slots == nullptr) return 0;
  const long long warps = (long long)T * nkv;
  const dim3 grid((unsigned)((warps + 7) / 8)), block(256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32)
    return launch_ex(value_norm_store_kernel<float>, grid, block, 0, s, 1, (const float*)proj, ld, k_off, v_off, nkv, kd, vd, eps,
                     norm, slots, (float*)kcache, (float*)vcache, page_size, T);
  if (dt == DT_BF16)
    return launch_ex(value_norm_store_kernel<bf16>, grid, block, 0, s, 1, (const bf16*)proj, ld, k_off, v_off, nkv, kd, vd, eps,
                     norm, slots, (bf16*)kcache, (bf16*)vcache, page_size, T);
  return ERR_BAD_DTYPE;
}

RLLM_API int rllm_talk_attention_simt(int dt, const void* q, long long q_ld, const void* kcache, const void* vcache,
                                      const int* token_seq, const int* positions, const int* block_table, long long bt_ld,
                                      const float* mix, const float* sinks, void* out, int T, int H, int G, int kd, int vd,
                                      int page_size, float scale, int window, int chunk, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || kd <= 0 || vd <= 0 || vd > 32 * MAX_VPL) return ERR_BAD_SIZE;
  const int rep = H / G;
  int warps = rep < 8 ? rep : 8;
  while (warps * MAX_HPW < H) ++warps;
  if (warps > 16) return ERR_BAD_SIZE;
  TalkArgs a;
  a.q = q; a.q_ld = q_ld; a.kcache = kcache; a.vcache = vcache; a.token_seq = token_seq; a.positions = positions;
  a.block_table = block_table; a.bt_ld = bt_ld; a.mix = mix; a.sinks = sinks; a.out = out; a.H = H; a.G = G; a.kd = kd;
  a.vd = vd; a.page_size = page_size; a.window = window; a.chunk = chunk; a.warps = warps; a.scale = scale;
  const int kvw = (kd + 1) > vd ? (kd + 1) : vd;
  const size_t smem = sizeof(float) * ((size_t)H * kd + (size_t)TK * kvw + 2 * (size_t)H * TK + (size_t)H * H + 2 * H);
  if (smem > 200 * 1024) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  static bool done_f[64], done_b[64];
  if (dt == DT_F32) {
    if (smem > 48 * 1024) { const int rc = allow_dynamic_smem(talk_attention_simt_kernel<float>, 200 * 1024, done_f); if (rc) return rc; }
    return launch_ex(talk_attention_simt_kernel<float>, dim3(T), dim3(32 * warps), smem, s, 1, a);
  }
  if (dt == DT_BF16) {
    if (smem > 48 * 1024) { const int rc = allow_dynamic_smem(talk_attention_simt_kernel<bf16>, 200 * 1024, done_b); if (rc) return rc; }
    return launch_ex(talk_attention_simt_kernel<bf16>, dim3(T), dim3(32 * warps), smem, s, 1, a);
  }
  return ERR_BAD_DTYPE;
}
