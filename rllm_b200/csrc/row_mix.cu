// Row-wise work of layers whose sublayers run side by side on one normed input, float arithmetic throughout.
//
// pair_embed: x[t] = table[id_t] + pair[r_t], then x / sqrt(mean(x^2) + eps) * w (w null: no norm). r_t is a hash of
//   the token and the one before it in its sequence, (prev * mul_prev + id * mul_cur) mod buckets, or row `buckets`
//   for a sequence's first token. The token before the first token of a portion is read from a slot of
//   per-request state; pair_embed_keep writes a portion's last token there afterwards (a kernel of its own: the
//   slot is read by another CTA of the first).
// combine: h[t] += sum_i c * w_i * a_i[t] / sqrt(mean(a_i[t]^2) + eps)   (up to two normed summands)
//                 + sum over up to three plain summands, each [T, parts, H] added in order of parts.
//   One pass over the row: the sum of a layer's sublayer outputs and the residual sum.
// glu_act: out[r, f] = act(gate, up) of in[r, f] and in[r, F + f]:
//   0: silu(g) * u     1: gelu_tanh(g) * u     2: g' = min(g, limit), u' = clamp(u, -limit, limit),
//                                                 g' * sigmoid(alpha g') * (u' + 1)
#include <cstdint>
#include <initializer_list>
#include "common.cuh"
using namespace rllm;

namespace {

__device__ __forceinline__ unsigned pair_row(long long prev, long long id, long long mul_prev, long long mul_cur, int buckets) {
  const unsigned long long b = (unsigned long long)buckets;
  auto md = [b](long long v) { long long r = v % (long long)b; return (unsigned long long)(r < 0 ? r + (long long)b : r); };
  return (unsigned)((md(prev) * md(mul_prev) + md(id) * md(mul_cur)) % b);
}

template <typename TW>
__global__ void pair_embed_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                  const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                  const int* __restrict__ state_slots, const int* __restrict__ prev_state,
                                  const TW* __restrict__ table, const TW* __restrict__ pair, const float* __restrict__ w,
                                  float eps, float* __restrict__ out, int H, int V, int buckets, long long mul_prev,
                                  long long mul_cur, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* prow = nullptr;
  if (pair != nullptr) {
    unsigned r = (unsigned)buckets;
    if (positions[t] > 0) {
      const int s = token_seq[t];
      int prev = 0;
      if (t > cu_q[s]) prev = ids[t - 1];
      else if (state_slots != nullptr && state_slots[s] >= 0) prev = prev_state[state_slots[s]];
      r = pair_row(prev, id, mul_prev, mul_cur, buckets);
    }
    prow = pair + (size_t)r * H;
  }
  const TW* trow = table + (size_t)id * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = to_f32(trow[i]) + (prow ? to_f32(prow[i]) : 0.f);
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  if (w == nullptr) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = row[i];
    return;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = row[i] * r * w[i];
}

__global__ void pair_embed_keep_kernel(const int* __restrict__ ids, const int* __restrict__ cu_q,
                                       const int* __restrict__ state_slots, int* __restrict__ prev_state, int S) {
  pdl_launch();
  pdl_wait();
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= S) return;
  const int slot = state_slots[s];
  if (slot >= 0 && cu_q[s + 1] > cu_q[s]) prev_state[slot] = ids[cu_q[s + 1] - 1];
}

// VEC 4: rows of a multiple of four numbers, read in 16-byte pieces (every row then starts on a 16-byte boundary).
template <int VEC>
__global__ void combine_kernel(float* __restrict__ h, const float* __restrict__ n0, const float* __restrict__ w0,
                               const float* __restrict__ n1, const float* __restrict__ w1, float coef, float eps,
                               const float* __restrict__ p0, int parts0, const float* __restrict__ p1, int parts1,
                               const float* __restrict__ p2, int parts2, int H) {
  pdl_launch();
  pdl_wait();
  struct V { float v[VEC]; };
  auto ld = [](const float* p) {
    V r;
    if (VEC == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; }
    else r.v[0] = *p;
    return r;
  };
  __shared__ float red[32];
  const size_t t = blockIdx.x;
  float r0 = 0.f, r1 = 0.f;
  if (n0) {
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
      const V x = ld(n0 + t * H + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss = fmaf(x.v[e], x.v[e], ss);
    }
    r0 = coef / sqrtf(block_sum(ss, red) / (float)H + eps);
  }
  if (n1) {
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
      const V x = ld(n1 + t * H + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss = fmaf(x.v[e], x.v[e], ss);
    }
    r1 = coef / sqrtf(block_sum(ss, red) / (float)H + eps);
  }
  for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
    V mix, ff;
#pragma unroll
    for (int e = 0; e < VEC; ++e) mix.v[e] = ff.v[e] = 0.f;
    if (n0) {
      const V x = ld(n0 + t * H + i), w = ld(w0 + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) mix.v[e] = x.v[e] * r0 * w.v[e];
    }
    if (n1) {
      const V x = ld(n1 + t * H + i), w = ld(w1 + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) mix.v[e] += x.v[e] * r1 * w.v[e];
    }
    auto sum = [&](const float* p, int parts, V& acc) {       // parts in their order, then added to acc
      if (!p) return;
      V m;
#pragma unroll
      for (int e = 0; e < VEC; ++e) m.v[e] = 0.f;
      const float* r = p + t * parts * H + i;
      for (int k = 0; k < parts; ++k) {
        const V x = ld(r + (size_t)k * H);
#pragma unroll
        for (int e = 0; e < VEC; ++e) m.v[e] += x.v[e];
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc.v[e] += m.v[e];
    };
    sum(p0, parts0, mix);
    V f1, f2;
#pragma unroll
    for (int e = 0; e < VEC; ++e) f1.v[e] = f2.v[e] = 0.f;
    sum(p1, parts1, f1);
    sum(p2, parts2, f2);
    const V hv = ld(h + t * H + i);
    float out[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) out[e] = hv.v[e] + (mix.v[e] + (f1.v[e] + f2.v[e]));
    if (VEC == 4) *reinterpret_cast<float4*>(h + t * H + i) = make_float4(out[0], out[1], out[2], out[3]);
    else h[t * H + i] = out[0];
  }
}

template <typename TI, typename TO>
__global__ void glu_act_kernel(const TI* __restrict__ in, long long ld, TO* __restrict__ out, int F, long long n, int kind,
                               float limit, float alpha, int block) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F;
    const int f = (int)(i % F);
    // gate columns then up columns, or blocks of `block` gate columns each followed by their up columns
    const int gc = block ? f / block * 2 * block + f % block : f, uc = block ? gc + block : F + f;
    float g = to_f32(in[r * ld + gc]), u = to_f32(in[r * ld + uc]);
    float y;
    if (kind == 0) {
      y = g / (1.f + expf(-g)) * u;
    } else if (kind == 1) {
      const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      y = 0.5f * g * (1.f + tanhf(z)) * u;
    } else {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      y = g / (1.f + expf(-alpha * g)) * (u + 1.f);
    }
    out[i] = from_f32<TO>(y);
  }
}

__global__ void add_bias_f32_kernel(float* __restrict__ y, const float* __restrict__ b, int N, long long n) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] += b[i % N];
}

inline unsigned blocks_for(long long n) { return (unsigned)((n + 255) / 256 > 65535 * 8 ? 65535 * 8 : (n + 255) / 256); }

}  // namespace

RLLM_API int rllm_pair_embed(const int* ids, const int* positions, const int* token_seq, const int* cu_q,
                             const int* state_slots, int* prev_state, const void* table, const void* pair, int dt,
                             const float* w, float eps, float* out, int T, int S, int H, int V, int buckets,
                             long long mul_prev, long long mul_cur, int* err, void* stream) {
  if (T <= 0) return 0;
  if (pair != nullptr && buckets <= 0) return ERR_BAD_SIZE;
  if ((size_t)H * sizeof(float) > 48 * 1024) return ERR_TOO_LARGE;
  const int threads = H >= 256 ? 256 : (H >= 128 ? 128 : 64);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = (size_t)H * sizeof(float);
  int rc;
  if (dt == DT_F32)
    rc = launch_ex(pair_embed_kernel<float>, dim3(T), dim3(threads), smem, s, 1, ids, positions, token_seq, cu_q, state_slots,
                   (const int*)prev_state, (const float*)table, (const float*)pair, w, eps, out, H, V, buckets, mul_prev, mul_cur, err);
  else if (dt == DT_BF16)
    rc = launch_ex(pair_embed_kernel<bf16>, dim3(T), dim3(threads), smem, s, 1, ids, positions, token_seq, cu_q, state_slots,
                   (const int*)prev_state, (const bf16*)table, (const bf16*)pair, w, eps, out, H, V, buckets, mul_prev, mul_cur, err);
  else return ERR_BAD_DTYPE;
  if (rc || pair == nullptr || state_slots == nullptr || prev_state == nullptr) return rc;
  return launch_ex(pair_embed_keep_kernel, dim3((S + 127) / 128), dim3(128), 0, s, 1, ids, cu_q, state_slots, prev_state, S);
}

RLLM_API int rllm_combine(float* h, const float* n0, const float* w0, const float* n1, const float* w1, float coef, float eps,
                          const float* p0, int parts0, const float* p1, int parts1, const float* p2, int parts2, int T,
                          int H, void* stream) {
  if (T <= 0) return 0;
  if ((n0 && !w0) || (n1 && !w1)) return ERR_BAD_SIZE;
  const int threads = H >= 1024 ? 256 : 128;
  bool aligned = H % 4 == 0;
  for (const void* q : {(const void*)h, (const void*)n0, (const void*)w0, (const void*)n1, (const void*)w1, (const void*)p0,
                        (const void*)p1, (const void*)p2})
    aligned = aligned && (reinterpret_cast<uintptr_t>(q) & 15) == 0;
  if (aligned)
    return launch_ex(combine_kernel<4>, dim3(T), dim3(threads), 0, (cudaStream_t)stream, 1, h, n0, w0, n1, w1, coef, eps, p0,
                     parts0, p1, parts1, p2, parts2, H);
  return launch_ex(combine_kernel<1>, dim3(T), dim3(threads), 0, (cudaStream_t)stream, 1, h, n0, w0, n1, w1, coef, eps, p0, parts0,
                   p1, parts1, p2, parts2, H);
}

RLLM_API int rllm_glu_act(const void* in, int in_dt, long long ld, void* out, int out_dt, int R, int F, int kind, float limit,
                          float alpha, int block, void* stream) {
  if (R <= 0 || F <= 0) return 0;
  if (kind < 0 || kind > 2 || block < 0 || (block && F % block)) return ERR_BAD_SIZE;
  const long long n = (long long)R * F;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 g(blocks_for(n)), b(256);
  if (in_dt == DT_F32 && out_dt == DT_F32)
    return launch_ex(glu_act_kernel<float, float>, g, b, 0, s, 1, (const float*)in, ld, (float*)out, F, n, kind, limit, alpha, block);
  if (in_dt == DT_F32 && out_dt == DT_BF16)
    return launch_ex(glu_act_kernel<float, bf16>, g, b, 0, s, 1, (const float*)in, ld, (bf16*)out, F, n, kind, limit, alpha, block);
  if (in_dt == DT_BF16 && out_dt == DT_BF16)
    return launch_ex(glu_act_kernel<bf16, bf16>, g, b, 0, s, 1, (const bf16*)in, ld, (bf16*)out, F, n, kind, limit, alpha, block);
  return ERR_BAD_DTYPE;
}

RLLM_API int rllm_add_bias_f32(float* y, const float* bias, int rows, int N, void* stream) {
  if (rows <= 0 || N <= 0) return 0;
  const long long n = (long long)rows * N;
  return launch_ex(add_bias_f32_kernel, dim3(blocks_for(n)), dim3(256), 0, (cudaStream_t)stream, 1, y, bias, N, n);
}
