// Routing of a mixture of experts, and the norm that follows a sublayer.
//
// moe_topk: per token, from float router logits [T, E] (plus a bias per expert, if given): scores = softmax over all
//   experts (score_fn 0), sigmoid of each logit by itself (score_fn 1), or the logits themselves, ranked as they are,
//   with the softmax over the chosen ones only as weights (score_fn 2); experts form
//   `groups` equal groups of neighbours, a group's score is its largest, only experts of the best `keep`
//   groups can be chosen (groups <= 1: no such limit); the `top` largest scores are chosen; their weights
//   are the scores themselves, or the scores divided by their sum (`renorm`). All in float. Of equal
//   scores the lower index wins.
// moe_plan: from the choices, the sorted row list the grouped product walks: per expert a segment of
//   (token, slot) pairs, cut into tiles of `tile_rows` rows. One CTA; a pair's place inside its expert's segment is
//   handed out by a counter, which changes where a row is computed, never its value.
// rmsnorm_add: residual[t] += w * y[t] / sqrt(mean(y[t]^2) + eps) with y[t] = sum over `parts` of
//   parts_in[t, p, :] in order (parts = 1: a plain post-norm; more: the combine of the chosen experts'
//   outputs, norm and residual sum in one pass). Float throughout.
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int MAX_E = 1024;      // experts a warp can rank (32 per lane)

__global__ void __launch_bounds__(128) moe_topk_kernel(const float* __restrict__ logits, int T, int E, int groups,
                                                       int keep, int top, int renorm, int score_fn,
                                                       const float* __restrict__ bias, int* __restrict__ idx,
                                                       float* __restrict__ wt) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];            // per warp: E scores, then E flags (1 allowed)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= T) return;
  float* s = sm + (size_t)warp * 2 * E;
  float* ok = s + E;
  const float* zr = logits + (size_t)t * E;
  auto z = [&](int e) { return bias ? zr[e] + bias[e] : zr[e]; };
  if (score_fn == 2) {
    for (int e = lane; e < E; e += 32) { s[e] = z(e); ok[e] = 1.f; }
  } else if (score_fn == 1) {
    for (int e = lane; e < E; e += 32) { s[e] = 1.f / (1.f + expf(-z(e))); ok[e] = 1.f; }
  } else {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, z(e));
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(z(e) - m); s[e] = v; sum += v; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E; e += 32) { s[e] *= inv; ok[e] = 1.f; }
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    // a group's score; then the best `keep` groups, one at a time
    for (int e = lane; e < E; e += 32) ok[e] = 0.f;
    __syncwarp();
    for (int r = 0; r < keep; ++r) {
      float best = -1.f; int bg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        if (ok[g * per] != 0.f) continue;                   // taken already
        float gm = 0.f;
        for (int i = 0; i < per; ++i) gm = fmaxf(gm, s[g * per + i]);
        if (gm > best) { best = gm; bg = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, bg, o);
        if (ob > best || (ob == best && og < bg)) { best = ob; bg = og; }
      }
      __syncwarp();
      for (int i = lane; i < per; i += 32) ok[bg * per + i] = 1.f;
      __syncwarp();
    }
  }
  float chosen_sum = 0.f, first_best = 0.f;
  for (int r = 0; r < top; ++r) {
    float best = -INFINITY; int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (ok[e] == 1.f && s[e] > best) { best = s[e]; be = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    __syncwarp();
    if (r == 0) first_best = best;
    // ranked logits: the weight is exp(logit - largest chosen logit), divided by the sum of these below
    const float val = score_fn == 2 ? expf(best - first_best) : best;
    if (lane == 0) { ok[be] = 2.f; idx[(size_t)t * top + r] = be; wt[(size_t)t * top + r] = val; }
    chosen_sum += val;
    __syncwarp();
  }
  if ((renorm || score_fn == 2) && lane < top) wt[(size_t)t * top + lane] /= chosen_sum;
}

// counts -> segments -> tiles -> places. n = T * top pairs, pair i = token i / top, slot i % top.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ idx, const float* __restrict__ wt, int n,
                                                        int top, int E, int tile_rows, int* __restrict__ rows_tok,
                                                        int* __restrict__ rows_dest, float* __restrict__ rows_scale,
                                                        int* __restrict__ tiles, int* __restrict__ n_tiles) {
  pdl_launch();
  pdl_wait();
  __shared__ int count[MAX_E], cursor[MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&count[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      cursor[e] = at;
      for (int r = 0; r < count[e]; r += tile_rows) {
        tiles[3 * nt] = e; tiles[3 * nt + 1] = at + r; tiles[3 * nt + 2] = min(tile_rows, count[e] - r);
        ++nt;
      }
      at += count[e];
    }
    *n_tiles = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int r = atomicAdd(&cursor[idx[i]], 1);
    rows_tok[r] = i / top;
    rows_dest[r] = i;
    rows_scale[r] = wt[i];
  }
}

__global__ void rmsnorm_add_kernel(const float* __restrict__ y, int parts, const float* __restrict__ w,
                                   float* __restrict__ residual, int H, float eps) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float row[];           // H floats
  __shared__ float red[32];
  const float* yr = y + (size_t)blockIdx.x * parts * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = yr[i];
    for (int p = 1; p < parts; ++p) v += yr[(size_t)p * H + i];
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)H + eps);
  float* hr = residual + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) hr[i] += row[i] * r * w[i];
}

__global__ void add_row_kernel(float* __restrict__ h, const float* __restrict__ v, int H, long long n) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    h[i] += v[i % H];
}

}  // namespace

RLLM_API int rllm_moe_topk(const float* logits, int T, int E, int groups, int keep, int top, int renorm, int score_fn,
                           const float* bias, int* idx, float* wt, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > MAX_E || top <= 0 || top > 32 || top > E || score_fn < 0 || score_fn > 2) return ERR_BAD_SIZE;
  if (score_fn == 2 && groups > 1) return ERR_BAD_SIZE;      // a group's score is a maximum of non-negative scores
  if (groups > 1 && (E % groups || keep <= 0 || keep > groups || top > (E / groups) * keep)) return ERR_BAD_SIZE;
  const size_t smem = (size_t)4 * 2 * E * sizeof(float);
  return launch_ex(moe_topk_kernel, dim3((T + 3) / 4), dim3(128), smem, (cudaStream_t)stream, 1, logits, T, E, groups,
                   keep, top, renorm, score_fn, bias, idx, wt);
}

// tiles: room for n / tile_rows + E entries of 3 ints.
RLLM_API int rllm_moe_plan(const int* idx, const float* wt, int T, int top, int E, int tile_rows, int* rows_tok,
                           int* rows_dest, float* rows_scale, int* tiles, int* n_tiles, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > MAX_E || top <= 0 || tile_rows <= 0) return ERR_BAD_SIZE;
  if ((long long)T * top > 2147483647LL) return ERR_TOO_LARGE;
  return launch_ex(moe_plan_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, 1, idx, wt, T * top, top, E, tile_rows,
                   rows_tok, rows_dest, rows_scale, tiles, n_tiles);
}

RLLM_API int rllm_rmsnorm_add(const float* y, int parts, const float* w, float* residual, int T, int H, float eps,
                              void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || parts <= 0 || (size_t)H * sizeof(float) > 200 * 1024) return ERR_BAD_SIZE;
  static bool done[64] = {};
  const int smem = H * (int)sizeof(float);
  if (smem > 48 * 1024) { const int rc = allow_dynamic_smem(rmsnorm_add_kernel, smem, done); if (rc) return rc; }
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  return launch_ex(rmsnorm_add_kernel, dim3(T), dim3(threads), (size_t)smem, (cudaStream_t)stream, 1, y, parts, w, residual, H, eps);
}

// h [T, H] += v [H] on every row.
RLLM_API int rllm_add_row(float* h, const float* v, int T, int H, void* stream) {
  if (T <= 0 || H <= 0) return 0;
  const long long n = (long long)T * H;
  const int blocks = (int)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  return launch_ex(add_row_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, 1, h, v, H, n);
}
