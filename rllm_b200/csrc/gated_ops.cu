// Row-wise work of layers whose sublayers are gated into the stream, and a gated recurrence whose gates read only
// the current token; float arithmetic throughout.
//
// gated_add: h[t, c] += sigmoid(g[t, c] + b[c]) * (c0 * y0[t, c] + c1 * y1[t, c])   (y1 may be absent)
//   the sublayer's output, the gate on it and the residual sum in one pass over the row.
// act_rows: out[r, f] = act(in[r, f]); 0: gelu in its tanh form, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
// mingru_scan: per channel c of a sequence, with z = sigmoid(pz + bz), u = px + bx,
//   cand = u + 1/2 where u >= 0 and sigmoid(u) where u < 0:
//       S_t = (1 - z_t) S_(t-1) + z_t cand_t,     out_t = S_t * silu(pg_t).
//   S lives in a float slot per request. A step is a linear map of S with a diagonal matrix, so long portions are
//   cut into chunks of CHUNK tokens that run side by side: a first kernel leaves every chunk's map (a, b) with
//   S_end = a S_start + b, a second one folds the maps of the chunks before its own, in order, and then walks its
//   chunk. The order of every sum depends on the portion's length and the chunk size only.
#include "common.cuh"
using namespace rllm;

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

template <bool TWO>
__global__ void gated_add_kernel(float* __restrict__ h, const float* __restrict__ g, long long ldg,
                                 const float* __restrict__ b, const float* __restrict__ y0, float c0,
                                 const float* __restrict__ y1, float c1, int W, long long n4) {
  pdl_launch();
  pdl_wait();
  const int w4 = W / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / w4;
    const int c = (int)(i % w4) * 4;
    const float4 gv = *reinterpret_cast<const float4*>(g + t * ldg + c);
    const float4 bv = b ? *reinterpret_cast<const float4*>(b + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 hv = *reinterpret_cast<float4*>(h + t * W + c);
    const float4 a = *reinterpret_cast<const float4*>(y0 + t * W + c);
    float4 y = make_float4(c0 * a.x, c0 * a.y, c0 * a.z, c0 * a.w);
    if (TWO) {
      const float4 d = *reinterpret_cast<const float4*>(y1 + t * W + c);
      y.x = fmaf(c1, d.x, y.x); y.y = fmaf(c1, d.y, y.y); y.z = fmaf(c1, d.z, y.z); y.w = fmaf(c1, d.w, y.w);
    }
    hv.x = fmaf(sigmoidf_(gv.x + bv.x), y.x, hv.x);
    hv.y = fmaf(sigmoidf_(gv.y + bv.y), y.y, hv.y);
    hv.z = fmaf(sigmoidf_(gv.z + bv.z), y.z, hv.z);
    hv.w = fmaf(sigmoidf_(gv.w + bv.w), y.w, hv.w);
    *reinterpret_cast<float4*>(h + t * W + c) = hv;
  }
}

__global__ void gated_add_any_kernel(float* __restrict__ h, const float* __restrict__ g, long long ldg,
                                     const float* __restrict__ b, const float* __restrict__ y0, float c0,
                                     const float* __restrict__ y1, float c1, int W, long long n) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / W;
    const int c = (int)(i % W);
    float y = c0 * y0[i];
    if (y1) y = fmaf(c1, y1[i], y);
    h[i] = fmaf(sigmoidf_(g[t * ldg + c] + (b ? b[c] : 0.f)), y, h[i]);
  }
}

__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TI, typename TO>
__global__ void act_rows_kernel(const TI* __restrict__ in, long long ld, TO* __restrict__ out, int F, long long n, int kind) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float z = to_f32(in[i / F * ld + i % F]);
    out[i] = from_f32<TO>(gelu_tanh_(z));
  }
}

// ---- the gated recurrence

constexpr int SCAN_THREADS = 128;

struct ScanArgs {
  const float* proj; long long ld;
  int z_off, x_off, g_off;
  const float* bz; const float* bx;
  const int* cu_q; const int* slots;
  float* state;            // [slots, R]
  int R, S, chunk;         // chunk 0: a sequence's portion is one piece
  float* ca; float* cb;    // [pieces, R]: the maps of the pieces (chunk > 0)
  float* s0;               // [S, R]: the state every sequence's first piece starts from (chunk > 0)
};

// Which sequence and which piece of its portion does block y have? Pieces are counted sequence by sequence.
__device__ __forceinline__ bool find_piece(const ScanArgs& p, int y, int& s, int& j, int& first_piece) {
  int acc = 0;
  for (s = 0; s < p.S; ++s) {
    const int len = p.cu_q[s + 1] - p.cu_q[s];
    const int n = p.chunk > 0 ? (len + p.chunk - 1) / p.chunk : (len > 0 ? 1 : 0);
    if (y < acc + n) { j = y - acc; first_piece = acc; return true; }
    acc += n;
  }
  return false;
}

__device__ __forceinline__ void gru_terms(float pz, float px, float bz, float bx, float& z, float& cand) {
  z = sigmoidf_(pz + bz);
  const float u = px + bx;
  cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
}

__global__ void __launch_bounds__(SCAN_THREADS) mingru_maps_kernel(const ScanArgs p) {
  pdl_launch();
  pdl_wait();
  const int c = blockIdx.x * SCAN_THREADS + threadIdx.x;
  int s, j, first;
  if (c >= p.R || !find_piece(p, blockIdx.y, s, j, first)) return;
  const int t0 = p.cu_q[s] + j * p.chunk, t1 = min(p.cu_q[s + 1], t0 + p.chunk);
  const float bz = p.bz ? p.bz[c] : 0.f, bx = p.bx ? p.bx[c] : 0.f;
  float a = 1.f, b = 0.f;
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const float* row = p.proj + (long long)t * p.ld;
    float z, cand;
    gru_terms(row[p.z_off + c], row[p.x_off + c], bz, bx, z, cand);
    a *= 1.f - z;
    b = fmaf(z, cand - b, b);
  }
  p.ca[(long long)blockIdx.y * p.R + c] = a;
  p.cb[(long long)blockIdx.y * p.R + c] = b;
  // the state as the step found it: the walk of a sequence's last piece overwrites the slot while others still start
  if (j == 0) {
    const int slot = p.slots ? p.slots[s] : -1;
    p.s0[(long long)s * p.R + c] = slot >= 0 ? p.state[(long long)slot * p.R + c] : 0.f;
  }
}

template <typename TO>
__global__ void __launch_bounds__(SCAN_THREADS) mingru_scan_kernel(const ScanArgs p, TO* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  const int c = blockIdx.x * SCAN_THREADS + threadIdx.x;
  int s, j, first;
  if (c >= p.R || !find_piece(p, blockIdx.y, s, j, first)) return;
  const int q0 = p.cu_q[s], q1 = p.cu_q[s + 1];
  const int t0 = p.chunk > 0 ? q0 + j * p.chunk : q0, t1 = p.chunk > 0 ? min(q1, t0 + p.chunk) : q1;
  const int slot = p.slots ? p.slots[s] : -1;
  const float bz = p.bz ? p.bz[c] : 0.f, bx = p.bx ? p.bx[c] : 0.f;
  float S = p.chunk > 0 ? p.s0[(long long)s * p.R + c] : (slot >= 0 ? p.state[(long long)slot * p.R + c] : 0.f);
  for (int i = 0; i < j; ++i)                                   // the pieces before this one, in order
    S = fmaf(p.ca[(long long)(first + i) * p.R + c], S, p.cb[(long long)(first + i) * p.R + c]);
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const float* row = p.proj + (long long)t * p.ld;
    float z, cand;
    gru_terms(row[p.z_off + c], row[p.x_off + c], bz, bx, z, cand);
    S = fmaf(z, cand - S, S);
    const float g = row[p.g_off + c];
    out[(long long)t * p.R + c] = from_f32<TO>(S * (g * sigmoidf_(g)));
  }
  if (t1 == q1 && slot >= 0) p.state[(long long)slot * p.R + c] = S;
}

inline unsigned blocks_for(long long n) { return (unsigned)((n + 255) / 256 > 65535 * 8 ? 65535 * 8 : (n + 255) / 256); }

}  // namespace

// h float [T, W] in place; g float rows of stride ldg (the gate's logits), b float [W] or null; y0, y1 float [T, W]
// (y1 null: one summand).
RLLM_API int rllm_gated_add(float* h, const float* g, long long ldg, const float* b, const float* y0, float c0,
                            const float* y1, float c1, int T, int W, void* stream) {
  if (T <= 0 || W <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const long long n = (long long)T * W;
  const bool vec = W % 4 == 0 && ldg % 4 == 0 && !(((uintptr_t)h | (uintptr_t)g | (uintptr_t)b | (uintptr_t)y0 | (uintptr_t)y1) & 15);
  if (vec) {
    const dim3 grid(blocks_for(n / 4)), blk(256);
    if (y1) return launch_ex(gated_add_kernel<true>, grid, blk, 0, s, 1, h, g, ldg, b, y0, c0, y1, c1, W, n / 4);
    return launch_ex(gated_add_kernel<false>, grid, blk, 0, s, 1, h, g, ldg, b, y0, c0, y1, c1, W, n / 4);
  }
  return launch_ex(gated_add_any_kernel, dim3(blocks_for(n)), dim3(256), 0, s, 1, h, g, ldg, b, y0, c0, y1, c1, W, n);
}

RLLM_API int rllm_act_rows(const void* in, int in_dt, long long ld, void* out, int out_dt, int R, int F, int kind,
                           void* stream) {
  if (R <= 0 || F <= 0) return 0;
  if (kind != 0) return ERR_BAD_SIZE;
  const long long n = (long long)R * F;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 g(blocks_for(n)), b(256);
  if (in_dt == DT_F32 && out_dt == DT_F32)
    return launch_ex(act_rows_kernel<float, float>, g, b, 0, s, 1, (const float*)in, ld, (float*)out, F, n, kind);
  if (in_dt == DT_F32 && out_dt == DT_BF16)
    return launch_ex(act_rows_kernel<float, bf16>, g, b, 0, s, 1, (const float*)in, ld, (bf16*)out, F, n, kind);
  if (in_dt == DT_BF16 && out_dt == DT_BF16)
    return launch_ex(act_rows_kernel<bf16, bf16>, g, b, 0, s, 1, (const bf16*)in, ld, (bf16*)out, F, n, kind);
  return ERR_BAD_DTYPE;
}

// proj float [T, ld] with the update gate's, the candidate's and the output gate's logits at columns z_off, x_off,
// g_off (R each); bz, bx float [R] or null; cu_q [S + 1]; slots [S] or null (the state starts at zero and is not
// kept); state float [slots, R]; out [T, R] of out_dt. chunk > 0: portions are cut into pieces of that many tokens,
// ca and cb float [T / chunk + S, R] hold the pieces' maps, s0 float [S, R] the states the step found.
RLLM_API int rllm_mingru_scan(const float* proj, long long ld, int z_off, int x_off, int g_off, const float* bz,
                              const float* bx, const int* cu_q, const int* slots, float* state, void* out, int out_dt,
                              int T, int S, int R, int chunk, float* ca, float* cb, float* s0, void* stream) {
  if (T <= 0 || S <= 0 || R <= 0) return 0;
  if (chunk < 0 || (chunk > 0 && (!ca || !cb || !s0))) return ERR_BAD_SIZE;
  const long long pieces = chunk > 0 ? (long long)T / chunk + S : S;
  if (pieces > 65535) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  const ScanArgs a = {proj, ld, z_off, x_off, g_off, bz, bx, cu_q, slots, state, R, S, chunk, ca, cb, s0};
  const dim3 grid((unsigned)((R + SCAN_THREADS - 1) / SCAN_THREADS), (unsigned)pieces), blk(SCAN_THREADS);
  if (chunk > 0) {
    const int rc = launch_ex(mingru_maps_kernel, grid, blk, 0, s, 1, a);
    if (rc) return rc;
  }
  if (out_dt == DT_F32) return launch_ex(mingru_scan_kernel<float>, grid, blk, 0, s, 1, a, (float*)out);
  if (out_dt == DT_BF16) return launch_ex(mingru_scan_kernel<bf16>, grid, blk, 0, s, 1, a, (bf16*)out);
  return ERR_BAD_DTYPE;
}
