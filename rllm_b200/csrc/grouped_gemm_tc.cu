// The ragged grouped product (csrc/grouped_gemm.cu) for long row lists in bfloat16 on the 5th-generation tensor
// cores: per tile of the routing plan (an expert, up to 128 sorted rows) and 128 weight rows of that expert
//   D[128 rows, 128 features] = A[rows, K] * W_e[features, K]^T
// with `tcgen05.mma` (M = 128, N = 128, K = 16 per instruction), both operands K-major in shared memory with the
// 128-byte swizzle, brought by TMA (`cp.async.bulk.tensor`, boxes of 64 of K x 128 rows) through a ring of three
// stages, the accumulator (128 lanes x 128 columns of float) in TMEM. The sorted rows are a matrix of their own
// ([rows of the plan, K]: the experts' inputs gathered by rllm_gather_rows_bf16, or the up product's output), so a
// tile is a plain box that starts at its first sorted row; rows of the box that belong to the next expert, or lie
// beyond the list, are computed and not stored. Likewise weight rows beyond an expert's N.
// Roles (192 threads): warp 0 one lane issues the copies, warp 1 allocates TMEM and one lane issues the products,
// warps 2..5 read the accumulator (a quarter of the lanes each, a row of the tile per thread) and store: relu^2 to
// bfloat16 rows in sorted order, or float rows scaled by the row's weight and scattered to the row's place.
// Every wait is bounded; a wait that runs out is recorded in `err` and the CTA drains and leaves.
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include "common.cuh"
#include "sm100.cuh"
using namespace rllm;
using namespace sm100;

namespace {

constexpr int TM = 128, TN = 128, TK = 64, UK = 16, STAGES = 3;
constexpr int OPERAND_BYTES = TM * TK * 2, STAGE_BYTES = 2 * OPERAND_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
enum : int { TEPI_RELU2 = 2, TEPI_F32 = 1, TEPI_SILU_GATED = 3 };

struct TcArgs {
  void* C; long long ldc;
  int N, K;
  const int* tiles; const int* n_tiles;
  const int* rows_out; const float* row_scale;
  int* err;
  int act; float limit, alpha;     // the gated epilogue: 0 silu(g) u, 1 gelu_tanh(g) u, 2 g' sigmoid(alpha g') (u' + 1), clamped
};

// act(g, u) of the gated epilogue, in float.
__device__ __forceinline__ float gated_act(float g, float u, int act, float limit, float alpha) {
  if (act == 0) return g / (1.f + __expf(-g)) * u;
  if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

template <int EPI>
__global__ void __launch_bounds__(192)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                       const TcArgs p) {
  pdl_launch();
  pdl_wait();                                   // the plan, the sorted rows: all come from kernels before
  if ((int)blockIdx.y >= *p.n_tiles) return;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int never_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int e = p.tiles[3 * blockIdx.y], row0 = p.tiles[3 * blockIdx.y + 1], rows = p.tiles[3 * blockIdx.y + 2];
  const int n0 = blockIdx.x * TN;
  const int n_kb = (p.K + TK - 1) / TK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_bar, 1);
    abort_flag = 0;
    never_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmap_a); prefetch_tensormap(&tmap_w); }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, TN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        if (i >= STAGES && !mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag)) {
          abort_flag = 1; if (p.err) record_failure(p.err, 11, blockIdx.y); break;
        }
        uint8_t* st = smem + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(st, &tmap_a, &full_bar[s], i * TK, row0);
        tma_load_2d(st + OPERAND_BYTES, &tmap_w, &full_bar[s], i * TK, e * p.N + n0);
        issued = i + 1;
      }
      if (abort_flag) {
        // let copies already issued land before the CTA's shared memory is given back
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          mbar_wait(&full_bar[i % STAGES], (uint32_t)(i / STAGES) & 1u, &never_flag, 200000000LL);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(TM, TN);
      const uint64_t d0 = umma_desc_sw128(smem_u32(smem));
      bool ok = true;
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], ph, &abort_flag)) { abort_flag = 1; if (p.err) record_failure(p.err, 12, blockIdx.y); ok = false; break; }
        tc_fence_after();
        const uint64_t da = d0 + (uint64_t)(s * (STAGE_BYTES >> 4));
        const uint64_t db = da + (uint64_t)(OPERAND_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < TK / UK; ++k) {
          const uint64_t koff = (uint64_t)(k * UK * 2 / 16);
          umma_bf16(tmem_base, da + koff, db + koff, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);             // the stage is free once these products have read it
      }
      if (ok) umma_commit(&acc_bar);
    }
  } else {
    // ---- epilogue warps 2..5: TMEM lanes [32 (warp & 3), +32), a row of the tile per thread
    bool ok = mbar_wait(&acc_bar, 0, &abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (!ok) { if (lane == 0) { abort_flag = 1; if (p.err) record_failure(p.err, 13, blockIdx.y); } }
    else {
      const int m = (warp & 3) * 32 + lane;
      const bool live = m < rows;
      const int r = row0 + (live ? m : 0);
      const float f = (live && p.row_scale) ? p.row_scale[r] : 1.f;
      const long long crow = live ? (p.rows_out ? p.rows_out[r] : r) : 0;
      const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
        if (!live) continue;
        const int n = n0 + c0;
        if (EPI == TEPI_F32) {
          float* c = (float*)p.C + crow * p.ldc + n;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            if (n + j < p.N)                    // N is a multiple of 8: four are in or out together
              *reinterpret_cast<float4*>(c + j) = make_float4(__uint_as_float(v[j]) * f, __uint_as_float(v[j + 1]) * f,
                                                              __uint_as_float(v[j + 2]) * f, __uint_as_float(v[j + 3]) * f);
        } else if (EPI == TEPI_SILU_GATED) {
          // the weight's rows come in blocks of 16 gate rows followed by their 16 up rows: these 32 columns hold
          // both halves of 16 outputs. The row's weight scales both linear results before the activation.
          if (n >= p.N) continue;                 // N is a multiple of 32
          bf16* c = (bf16*)p.C + crow * p.ldc + n / 2;
#pragma unroll
          for (int j = 0; j < 16; j += 8) {
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float g0 = __uint_as_float(v[j + 2 * q]) * f, g1 = __uint_as_float(v[j + 2 * q + 1]) * f;
              const float u0 = __uint_as_float(v[16 + j + 2 * q]) * f, u1 = __uint_as_float(v[16 + j + 2 * q + 1]) * f;
              __nv_bfloat162 h = __floats2bfloat162_rn(gated_act(g0, u0, p.act, p.limit, p.alpha), gated_act(g1, u1, p.act, p.limit, p.alpha));
              o[q] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(c + j) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          bf16* c = (bf16*)p.C + crow * p.ldc + n;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (n + j >= p.N) continue;
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float a = fmaxf(__uint_as_float(v[j + 2 * q]), 0.f), b = fmaxf(__uint_as_float(v[j + 2 * q + 1]), 0.f);
              __nv_bfloat162 h = __floats2bfloat162_rn(a * a * f, b * b * f);
              o[q] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(c + j) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TN); }
}

__global__ void gather_rows_bf16_kernel(const bf16* __restrict__ x, long long ldx, const int* __restrict__ idx,
                                        bf16* __restrict__ out, int n_rows, int K) {
  pdl_launch();
  pdl_wait();
  const int per = K / 8;                        // 16-byte pieces of a row
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)n_rows * per;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / per), c = (int)(i % per);
    reinterpret_cast<uint4*>(out + (long long)r * K)[c] = reinterpret_cast<const uint4*>(x + (long long)idx[r] * ldx)[c];
  }
}

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_mu;

int get_encoder() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return -5;
  }
  g_encode = (EncodeTiledFn)fn;
  return 0;
}

// bfloat16 matrix [rows, cols], row stride ld elements; boxes of 64 columns x 128 rows, 128-byte swizzle, zeros
// outside
int make_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, long long ld) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TK, (cuuint32_t)TM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -5;
}

template <int EPI>
int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, const TcArgs& p, dim3 grid, cudaStream_t s) {
  static bool done[64] = {};
  if (allow_dynamic_smem(grouped_gemm_tc_kernel<EPI>, SMEM_BYTES, done)) return -5;
  return launch_ex(grouped_gemm_tc_kernel<EPI>, grid, dim3(192), (size_t)SMEM_BYTES, s, 1, ma, mw, p);
}

}  // namespace

// Can rllm_grouped_gemm_tc take a product of these sizes? (16-byte aligned rows, whole groups of 8 features)
RLLM_API int rllm_grouped_gemm_tc_supported(long long lda, int N, int K) {
  return K % 8 == 0 && lda % 8 == 0 && N % 8 == 0 && K >= 64;
}

// A: bfloat16 [a_rows, K], row stride lda: the plan's sorted rows. W: bfloat16 [E, N, K]. The plan (tiles of up to 128
// rows) as for rllm_grouped_gemm_ragged. epi 2: C bfloat16 [a_rows, N] = relu(.)^2 in sorted order; epi 1: C float,
// row rows_out[r] = row_scale[r] * (.); epi 3: W's rows in blocks of 16 gate rows and their 16 up rows (N a multiple
// of 32), C bfloat16 [a_rows, N / 2] = act(f g, f u) with f = row_scale[r] (1 without) and act by `act`, `limit`, `alpha`:
// 0 silu(g) u, 1 gelu_tanh(g) u, 2 g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit).
// err: one int on the device for a wait that ran out, or null.
RLLM_API int rllm_grouped_gemm_tc(int epi, const void* A, long long lda, long long a_rows, const void* W, int E, int N,
                                  int K, void* C, long long ldc, const int* tiles, const int* n_tiles, int max_tiles,
                                  const int* rows_out, const float* row_scale, int* err, int act, float limit, float alpha,
                                  void* stream) {
  if (max_tiles <= 0 || a_rows <= 0) return 0;
  if (!rllm_grouped_gemm_tc_supported(lda, N, K) || !tiles || !n_tiles || E <= 0) return ERR_BAD_SIZE;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)C & 15) || ldc % 8) return ERR_BAD_ALIGN;
  if (max_tiles > 65535 || (long long)E * N > 2147483647LL) return ERR_TOO_LARGE;
  if (get_encoder()) return -5;
  CUtensorMap ma, mw;
  if (make_map(&ma, A, a_rows, K, lda) || make_map(&mw, W, (long long)E * N, K, K)) return -5;
  if (act < 0 || act > 2) return ERR_BAD_SIZE;
  TcArgs p = {C, ldc, N, K, tiles, n_tiles, rows_out, row_scale, err, act, limit, alpha};
  dim3 grid((N + TN - 1) / TN, max_tiles, 1);
  if (epi == TEPI_RELU2) return launch_tc<TEPI_RELU2>(ma, mw, p, grid, (cudaStream_t)stream);
  if (epi == TEPI_F32) return launch_tc<TEPI_F32>(ma, mw, p, grid, (cudaStream_t)stream);
  if (epi == TEPI_SILU_GATED) {
    if (N % 32) return ERR_BAD_SIZE;
    return launch_tc<TEPI_SILU_GATED>(ma, mw, p, grid, (cudaStream_t)stream);
  }
  return ERR_BAD_SIZE;
}

// out[r, :] = x[idx[r], :] for bfloat16 rows of K (a multiple of 8) numbers.
RLLM_API int rllm_gather_rows_bf16(const void* x, long long ldx, const int* idx, void* out, int n_rows, int K,
                                   void* stream) {
  if (n_rows <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return ERR_BAD_ALIGN;
  const long long total = (long long)n_rows * (K / 8);
  const int blocks = (int)((total + 255) / 256 < 4736 ? (total + 255) / 256 : 4736);
  return launch_ex(gather_rows_bf16_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, 1, (const bf16*)x, ldx, idx,
                   (bf16*)out, n_rows, K);
}
