// Grouped-query attention with the extras some designs put around it, over the paged cache:
//
//   * keys and values of different sizes per head (kd, vd): the value pages are [page][kv head][offset][vd];
//   * a per-head RMS norm of queries and keys (one weight of kd numbers for all heads) before the rotation;
//   * a rotation of the first `rot` dimensions of a head, dimension i paired with i + rot/2, the rest passing;
//   * a mask that is causal and, besides, a window (the last `window` positions) and/or a block rule (only
//     the positions of the query's own block of `chunk` positions, blocks counted from position 0);
//   * kept first keys: with `keep_first` > 0 a query also sees every position below that number, whatever the window says;
//   * a sink: a learned number per head that joins the softmax's denominator with no key and no value;
//   * sigmoid weights in place of the softmax (`sigmoid` != 0): a visible key's weight is
//     sigmoid(score + bias[head]), not normalised over the keys (`sinks` then holds the biases);
//   * an output gate: head h's output times sigmoid(gate[t, h]).
//
// qk_norm_rope_store prepares a step's queries (in place) and writes its keys and values into their pages, the values
// optionally mixed with another layer's of the same tokens on the way: v <- (1 - lam) v + lam v_first (float, one rounding);
// sink_attention_simt is the attention itself on the CUDA cores, in float whatever the storage type (the
// 32-bit path, and sizes the tensor-core kernel refuses); sink_attention_mma (sink_attention_mma.cuh) is the
// bfloat16 kernel on the tensor cores. A query's result depends on its position and the cache's contents
// only: keys are walked in position order in fixed tiles counted from the first visible key's tile.
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int MAX_D = 256;

// One warp per (token, q head | k head | v head). Norm and rotation in float; q goes back into `proj` in place.
template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_rope_store_kernel(T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int n_tokens, int nh,
                          int nkv, int kd, int vd, int rot, const float* __restrict__ wq, const float* __restrict__ wk,
                          float eps, const float* __restrict__ table, const int* __restrict__ slots,
                          T* __restrict__ kcache, T* __restrict__ vcache, int page_size, const T* __restrict__ vfirst,
                          long long ldf, const float* __restrict__ lam) {
  pdl_launch();
  pdl_wait();
  __shared__ float xs[4][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = nh + 2 * nkv;
  const long long gw = (long long)blockIdx.x * 4 + warp;
  if (gw >= (long long)n_tokens * per) return;
  const int t = (int)(gw / per), u = (int)(gw % per);
  T* row = proj + (long long)t * ld;
  const int slot = slots ? slots[t] : -1;
  if (u >= nh + nkv) {                       // a value head: a copy into its page
    if (slot < 0 || !vcache) return;
    const int g = u - nh - nkv;
    const T* src = row + v_off + g * vd;
    T* dst = vcache + (((long long)(slot / page_size) * nkv + g) * page_size + slot % page_size) * vd;
    if (vfirst) {
      const float l = lam[0];
      const T* first = vfirst + (long long)t * ldf + g * vd;
      for (int d = lane; d < vd; d += 32) dst[d] = from_f32<T>(fmaf(l, to_f32(first[d]), (1.f - l) * to_f32(src[d])));
    } else {
      for (int d = lane; d < vd; d += 32) dst[d] = src[d];
    }
    return;
  }
  const bool is_q = u < nh;
  if (!is_q && (slot < 0 || !kcache)) return;
  T* src = is_q ? row + q_off + u * kd : row + k_off + (u - nh) * kd;
  const float* w = is_q ? wq : wk;
  float ss = 0.f;
  for (int d = lane; d < kd; d += 32) { const float v = to_f32(src[d]); xs[warp][d] = v; ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  __syncwarp();
  if (w) {
    const float r = 1.f / sqrtf(ss / (float)kd + eps);
    for (int d = lane; d < kd; d += 32) xs[warp][d] = xs[warp][d] * r * w[d];
    __syncwarp();
  }
  T* dst = is_q ? src : kcache + (((long long)(slot / page_size) * nkv + (u - nh)) * page_size + slot % page_size) * kd;
  const int half = rot / 2;
  const float* cs = table ? table + (long long)t * half * 2 : nullptr;
  for (int d = lane; d < kd; d += 32) {
    float v = xs[warp][d];
    if (cs && d < half) v = v * cs[2 * d] - xs[warp][d + half] * cs[2 * d + 1];
    else if (cs && d < rot) v = v * cs[2 * (d - half)] + xs[warp][d - half] * cs[2 * (d - half) + 1];
    dst[d] = from_f32<T>(v);
  }
}

// The same for bfloat16 rows in 16-byte pieces (head sizes multiples of 8, rotated width a multiple of 16): LPH lanes
// a head, each with one piece of 8 numbers and, inside the rotated part, a second look at the piece it pairs
// with; the sum of squares crosses the head's lanes by shuffles. Nothing is staged: all loads of a warp are
// issued before its first store (queries are rewritten in place).
template <int LPH>
__global__ void __launch_bounds__(128)
qk_norm_rope_store_vec_kernel(bf16* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int n_tokens, int nh,
                              int nkv, int kd, int vd, int rot, const float* __restrict__ wq, const float* __restrict__ wk,
                              float eps, const float* __restrict__ table, const int* __restrict__ slots,
                              bf16* __restrict__ kcache, bf16* __restrict__ vcache, int page_size,
                              const bf16* __restrict__ vfirst, long long ldf, const float* __restrict__ lam) {
  pdl_launch();
  pdl_wait();
  constexpr int HPW = 32 / LPH;                      // heads a warp
  const int lane = threadIdx.x & 31;
  const int per = nh + 2 * nkv;
  const long long item = ((long long)blockIdx.x * 4 + (threadIdx.x >> 5)) * HPW + lane / LPH;
  const int c = lane % LPH;
  const bool live = item < (long long)n_tokens * per;
  const int t = live ? (int)(item / per) : 0, u = live ? (int)(item % per) : 0;
  bf16* row = proj + (long long)t * ld;
  const int slot = (live && slots) ? slots[t] : -1;
  const bool is_q = u < nh, is_v = u >= nh + nkv;
  const int size = is_v ? vd : kd;
  const bool mine = live && c * 8 < size && (is_q || slot >= 0);
  bf16* src = is_q ? row + q_off + u * kd : (is_v ? row + v_off + (u - nh - nkv) * vd : row + k_off + (u - nh) * kd);
  const int half = rot / 2;
  const bool turns = mine && !is_v && table && c * 8 < rot;
  const int cp = c * 8 < half ? c + half / 8 : c - half / 8;             // the piece this one pairs with
  uint4 own = make_uint4(0, 0, 0, 0), other = make_uint4(0, 0, 0, 0);
  if (mine) own = *reinterpret_cast<const uint4*>(src + c * 8);
  if (turns) other = *reinterpret_cast<const uint4*>(src + cp * 8);
  const bool mixes = mine && is_v && vfirst;          // a value piece: the other layer's piece of the same token and head
  if (mixes) other = *reinterpret_cast<const uint4*>(vfirst + (long long)t * ldf + (u - nh - nkv) * vd + c * 8);
  float x[8], y[8];
  {
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&own);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&other);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(a[i]), g = __bfloat1622float2(b[i]);
      x[2 * i] = f.x; x[2 * i + 1] = f.y; y[2 * i] = g.x; y[2 * i + 1] = g.y;
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float* w = is_q ? wq : wk;
  if (mine && !is_v && w) {
    const float r = 1.f / sqrtf(ss / (float)kd + eps);
    const float4 w0 = reinterpret_cast<const float4*>(w + c * 8)[0], w1 = reinterpret_cast<const float4*>(w + c * 8)[1];
    x[0] *= r * w0.x; x[1] *= r * w0.y; x[2] *= r * w0.z; x[3] *= r * w0.w;
    x[4] *= r * w1.x; x[5] *= r * w1.y; x[6] *= r * w1.z; x[7] *= r * w1.w;
    if (turns) {
      const float4 p0 = reinterpret_cast<const float4*>(w + cp * 8)[0], p1 = reinterpret_cast<const float4*>(w + cp * 8)[1];
      y[0] *= r * p0.x; y[1] *= r * p0.y; y[2] *= r * p0.z; y[3] *= r * p0.w;
      y[4] *= r * p1.x; y[5] *= r * p1.y; y[6] *= r * p1.z; y[7] *= r * p1.w;
    }
  }
  if (mixes) {
    const float l = lam[0];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = fmaf(l, y[i], (1.f - l) * x[i]);
  }
  if (turns) {
    const int f0 = (c * 8) % half;
    const float4* cs = reinterpret_cast<const float4*>(table + ((long long)t * half + f0) * 2);
    const float sg = c * 8 < half ? -1.f : 1.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = cs[i];                           // (cos, sin) of two frequencies
      x[2 * i] = x[2 * i] * v.x + sg * y[2 * i] * v.y;
      x[2 * i + 1] = x[2 * i + 1] * v.z + sg * y[2 * i + 1] * v.w;
    }
  }
  __syncwarp();                                         // every load of the warp is done: queries may be rewritten
  if (!mine) return;
  bf16* dst = src;
  if (!is_q) {
    const int g = is_v ? u - nh - nkv : u - nh;
    dst = (is_v ? vcache : kcache) + (((long long)(slot / page_size) * nkv + g) * page_size + slot % page_size) * size;
  }
  uint4 o;
  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) ob[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst + c * 8) = o;
}

constexpr int WARPS = 4;

template <typename T> struct Vec16 {};
template <> struct Vec16<float> { static constexpr int N = 4; typedef float4 V; };
template <> struct Vec16<bf16> { static constexpr int N = 8; typedef uint4 V; };

__device__ __forceinline__ float dot_vec(const float4& k, const float* q) {
  return k.x * q[0] + k.y * q[1] + k.z * q[2] + k.w * q[3];
}
__device__ __forceinline__ float dot_vec(const uint4& k, const float* q) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&k);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    s = fmaf(f.x, q[2 * i], s);
    s = fmaf(f.y, q[2 * i + 1], s);
  }
  return s;
}

// One warp per (query token, query head); 32 keys a round in position order, running maximum and sum. The
// sink opens the running softmax as a key of score `sink` and value zero.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
sink_attention_simt_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ kcache,
                           const T* __restrict__ vcache, T* __restrict__ out, long long out_stride,
                           const int* __restrict__ token_seq, const int* __restrict__ positions,
                           const int* __restrict__ block_table, int bt_stride, int n_tokens, int nh, int nkv, int kd,
                           int vd, int page_size, float scale, int window, int chunk, const float* __restrict__ sinks,
                           const float* __restrict__ gate, int gate_ld, int keep_first, int sigmoid) {
  pdl_launch();
  pdl_wait();
  __shared__ float qs[WARPS][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * WARPS + warp;
  if (gw >= (long long)n_tokens * nh) return;
  const int t = (int)(gw / nh), h = (int)(gw % nh);
  const int kvh = h / (nh / nkv);
  const int seq = token_seq[t];
  const int pos = positions[t];
  int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (chunk > 0) start = max(start, pos / chunk * chunk);
  const int* bt = block_table + (size_t)seq * bt_stride;

  const T* qp = q + (size_t)t * q_stride + (size_t)h * kd;
  for (int d = lane; d < kd; d += 32) qs[warp][d] = to_f32(qp[d]) * scale;
  __syncwarp();

  constexpr int NACC = MAX_D / 32;
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  float m = (sinks && !sigmoid) ? sinks[h] : -INFINITY, l = (sinks && !sigmoid) ? 1.f : 0.f;
  const float sbias = (sinks && sigmoid) ? sinks[h] : 0.f;

  typedef typename Vec16<T>::V V;
  constexpr int VN = Vec16<T>::N;

  // the kept first keys that lie before the window's first key, then the window's keys
  const int kept = min(keep_first, start);
  for (int seg = kept > 0 ? 0 : 1; seg < 2; ++seg) {
  const int seg_lo = seg ? start : 0, seg_hi = seg ? pos : kept - 1;
  for (int base = seg_lo; base <= seg_hi; base += 32) {
    const int j = base + lane;
    bool valid = j <= seg_hi;
    float s = -INFINITY;
    long long slot = 0;
    const int page = valid ? bt[j / page_size] : -1;
    valid = valid && page >= 0;
    if (valid) {
      slot = ((long long)page * nkv + kvh) * page_size + (j % page_size);
      float dsum = 0.f;
      if (kd % VN == 0) {                    // rows start on 16 bytes
        const V* kp = reinterpret_cast<const V*>(kcache + slot * kd);
        for (int c = 0; c < kd / VN; ++c) dsum += dot_vec(kp[c], &qs[warp][c * VN]);
      } else {
        const T* kp = kcache + slot * kd;
        for (int d = 0; d < kd; ++d) dsum = fmaf(to_f32(kp[d]), qs[warp][d], dsum);
      }
      s = dsum;
    }
    float p, m_new = m;
    if (sigmoid) {
      p = valid ? 1.f / (1.f + expf(-(s + sbias))) : 0.f;
    } else {
      m_new = fmaxf(m, warp_max(s));
      p = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);
      l = l * corr + warp_sum(p);
#pragma unroll
      for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    }
    const int cnt = min(32, seg_hi - base + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long sj = __shfl_sync(0xffffffffu, slot, jj);
      const T* vp = vcache + sj * vd;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) acc[i] = fmaf(pj, to_f32(vp[d]), acc[i]);
      }
    }
    m = m_new;
  }
  }
  float f = sigmoid ? 1.f : (l > 0.f ? 1.f / l : 0.f);
  if (gate) f *= 1.f / (1.f + expf(-gate[(size_t)t * gate_ld + h]));
  T* op = out + (size_t)t * out_stride + (size_t)h * vd;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < vd) op[d] = from_f32<T>(acc[i] * f);
  }
}

}  // namespace

#include "sink_attention_mma.cuh"

// proj [T, ld]: q heads at q_off (nh x kd), k heads at k_off (nkv x kd), v heads at v_off (nkv x vd). wq, wk: float
// [kd] or null (no norm). table: float [T, rot/2, 2] (cos, sin) or null (no rotation). slots [T] (-1: the
// token's key and value are not stored) or null; kcache [pages, nkv, page, kd], vcache [pages, nkv, page, vd]. vfirst
// (rows of proj's type with stride ldf: nkv heads of vd per token) with lam (one float on the device) or both null.
RLLM_API int rllm_qk_norm_rope_store(int dt, void* proj, long long ld, int q_off, int k_off, int v_off, int n_tokens,
                                     int nh, int nkv, int kd, int vd, int rot, const float* wq, const float* wk,
                                     float eps, const float* table, const int* slots, void* kcache, void* vcache,
                                     int page_size, const void* vfirst, long long ldf, const float* lam, void* stream) {
  if (n_tokens <= 0) return 0;
  if (kd <= 0 || kd > MAX_D || vd <= 0 || vd > MAX_D || nh <= 0 || nkv <= 0 || rot < 0 || rot > kd || rot % 2 ||
      page_size <= 0)
    return ERR_BAD_SIZE;
  const long long warps = (long long)n_tokens * (nh + 2 * nkv);
  const long long blocks = (warps + 3) / 4;
  if (blocks > 2147483647LL) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (rot == 0) table = nullptr;
  if ((vfirst != nullptr) != (lam != nullptr)) return ERR_BAD_SIZE;
  if (dt == DT_F32)
    return launch_ex(qk_norm_rope_store_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, s, 1, (float*)proj, ld, q_off,
                     k_off, v_off, n_tokens, nh, nkv, kd, vd, rot, wq, wk, eps, table, slots, (float*)kcache,
                     (float*)vcache, page_size, (const float*)vfirst, ldf, lam);
  const bool vec = dt == DT_BF16 && kd % 8 == 0 && vd % 8 == 0 && rot % 16 == 0 && ld % 8 == 0 && q_off % 8 == 0 &&
                   k_off % 8 == 0 && v_off % 8 == 0 && !((uintptr_t)proj & 15) && !((uintptr_t)kcache & 15) &&
                   !((uintptr_t)vcache & 15) && !((uintptr_t)wq & 15) && !((uintptr_t)wk & 15) && !((uintptr_t)table & 15) &&
                   !((uintptr_t)vfirst & 15) && ldf % 8 == 0 &&
                   (slots != nullptr) == (kcache != nullptr && vcache != nullptr);
  if (vec) {
    const int pieces = (kd > vd ? kd : vd) / 8;
    int lph = 1;
    while (lph < pieces) lph *= 2;
    const long long items = (long long)n_tokens * (nh + 2 * nkv);
    const long long vblocks = (items + 4 * (32 / lph) - 1) / (4 * (32 / lph));
    if (vblocks > 2147483647LL) return ERR_TOO_LARGE;
#define GO(L) return launch_ex(qk_norm_rope_store_vec_kernel<L>, dim3((unsigned)vblocks), dim3(128), 0, s, 1, (bf16*)proj, ld, \
                               q_off, k_off, v_off, n_tokens, nh, nkv, kd, vd, rot, wq, wk, eps, table, slots, (bf16*)kcache,  \
                               (bf16*)vcache, page_size, (const bf16*)vfirst, ldf, lam)
    switch (lph) {
      case 1: GO(1);
      case 2: GO(2);
      case 4: GO(4);
      case 8: GO(8);
      case 16: GO(16);
      default: GO(32);
    }
#undef GO
  }
  if (dt == DT_BF16)
    return launch_ex(qk_norm_rope_store_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, s, 1, (bf16*)proj, ld, q_off,
                     k_off, v_off, n_tokens, nh, nkv, kd, vd, rot, wq, wk, eps, table, slots, (bf16*)kcache,
                     (bf16*)vcache, page_size, (const bf16*)vfirst, ldf, lam);
  return ERR_BAD_DTYPE;
}

// q [T, ...] row stride q_stride, head h at h * kd; out [T, ...] head h at h * vd. sinks: float [nh] or null (with
// `sigmoid` the biases of the sigmoid weights); gate: float logits [T, gate_ld] or null. window, chunk, keep_first: 0 = none.
RLLM_API int rllm_sink_attention_simt(int dt, const void* q, long long q_stride, const void* kcache, const void* vcache,
                                      void* out, long long out_stride, const int* token_seq, const int* positions,
                                      const int* block_table, int bt_stride, int n_tokens, int nh, int nkv, int kd, int vd,
                                      int page_size, float scale, int window, int chunk, const float* sinks,
                                      const float* gate, int gate_ld, int keep_first, int sigmoid, void* stream) {
  if (n_tokens <= 0) return 0;
  if (kd <= 0 || kd > MAX_D || vd <= 0 || vd > MAX_D || nkv <= 0 || nh % nkv || page_size <= 0 || keep_first < 0)
    return ERR_BAD_SIZE;
  const long long warps = (long long)n_tokens * nh;
  const long long blocks = (warps + WARPS - 1) / WARPS;
  if (blocks > 2147483647LL) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32)
    return launch_ex(sink_attention_simt_kernel<float>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, s, 1, (const float*)q,
                     q_stride, (const float*)kcache, (const float*)vcache, (float*)out, out_stride, token_seq, positions,
                     block_table, bt_stride, n_tokens, nh, nkv, kd, vd, page_size, scale, window, chunk, sinks, gate,
                     gate_ld, keep_first, sigmoid);
  if (dt == DT_BF16)
    return launch_ex(sink_attention_simt_kernel<bf16>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, s, 1, (const bf16*)q,
                     q_stride, (const bf16*)kcache, (const bf16*)vcache, (bf16*)out, out_stride, token_seq, positions,
                     block_table, bt_stride, n_tokens, nh, nkv, kd, vd, page_size, scale, window, chunk, sinks, gate,
                     gate_ld, keep_first, sigmoid);
  return ERR_BAD_DTYPE;
}
