// The attention of sink_attention.cu in bfloat16 on the tensor cores (`mma.sync` m16n8k16, float accumulators and
// float softmax), for prompt portions, single decoded tokens and any mix of them in one launch.
//
// A CTA (four warps) takes one tile of 64 rows of one sequence and one kv head; a row is a (query token, query
// head of the kv head's group) pair, so the heads that share keys share their tiles: a single decoded token
// with 16 heads a kv head fills a warp's 16 rows. Which sequence and tile a CTA has it finds from the row
// ranges on the device (the grid is the step's upper bound of tiles), so nothing of the launch depends on
// what the host cannot know when a decode graph is captured. Keys come in tiles of 64, aligned to 64 from
// position 0, copied through the block table by `cp.async` (16 bytes a copy, one tile in flight beside the one at work); only the
// tiles between the first key any row sees (window and block rule) and the last row's own position are
// walked (with kept first keys: the tiles of those keys first, then the window's), keys outside a row's mask get
// -inf. The sink opens a row's running softmax as a key of score `sink` and value zero. SIG: a visible key's weight
// is sigmoid(score + bias[head]) and nothing is normalised; the running maximum then stays 0 and the denominator 1,
// so that the joins of parts below are plain sums. With `splits` > 1 the CTAs of grid.z share a tile's key tiles in fixed ranges and write
// unnormalised parts (sum, maximum, denominator) that sink_attention_merge joins in range order; the sink goes
// with the first range, the output gate with whoever writes the result. Head sizes are padded with zeros in
// shared memory to DP (64 or 128) numbers. Steps whose sequences bring at most 16 rows each (decoding) take the
// FEW form of the kernel: see there.
#pragma once

namespace sinkmma {

constexpr int ROWS = 64, KEYS = 64, THREADS = 128, STAGES = 2;      // three stages measured level with two

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ float fast_exp2(float x) {          // exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {           // 1 / inf = 0; relative error about 2^-23
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

struct Args {
  const bf16* q; long long q_stride;
  const bf16* kcache; const bf16* vcache;
  bf16* out; long long out_stride;
  const int* positions; const int* cu_q; const int* block_table; int bt_stride;
  int num_seqs, nh, nkv, kd, vd, page_size;
  float scale_log2;            // scale * log2(e)
  int window, chunk;
  const float* sinks; const float* gate; int gate_ld;
  int splits; float* pacc; float* pml;
  int page_shift;              // log2(page_size), or -1 when it is no power of two
  int keep_first;              // positions below this number are seen whatever the window says
};

__device__ __forceinline__ int first_key(int pos, int window, int chunk) {
  int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (chunk > 0) start = max(start, pos / chunk * chunk);
  return start;
}

// FEW: the step's sequences bring at most 16 rows each (single tokens with up to 16 heads a kv head). The four warps
// then all hold the tile's 16 rows and split each tile's 64 keys between them (16 keys a warp), each with a running
// softmax of its own; the four are joined in warp order through shared memory at the end.
template <int DP, bool FEW, bool SIG>
__global__ void __launch_bounds__(THREADS) sink_attention_mma_kernel(const Args p) {
  pdl_launch();
  pdl_wait();
  constexpr int LD = DP + 8;                       // padded row of a key or value tile, in elements
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw);    // [STAGES][KEYS][LD]
  bf16* Vs = Ks + STAGES * KEYS * LD;              // [STAGES][KEYS][LD]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Gq = p.nh / p.nkv, g = blockIdx.y, z = blockIdx.z;

  // which sequence, which tile of its rows. FEW: every sequence has one tile. Else 32 sequences a round: each lane
  // counts one sequence's tiles, a warp scan finds the one that holds tile blockIdx.x (every warp for itself).
  int b = blockIdx.x, s = -1;
  if (FEW) {
    if (b < p.num_seqs) { s = b; b = 0; }
  } else {
    int base = 0;
    for (int s0 = 0; s0 < p.num_seqs; s0 += 32) {
      const int i = s0 + lane;
      const int nt = i < p.num_seqs ? ((p.cu_q[i + 1] - p.cu_q[i]) * Gq + ROWS - 1) / ROWS : 0;
      int inc = nt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      const int total = __shfl_sync(0xffffffffu, inc, 31);
      if (b < base + total) {
        const int l = __ffs(__ballot_sync(0xffffffffu, b < base + inc)) - 1;
        s = s0 + l;
        b -= base + __shfl_sync(0xffffffffu, inc - nt, l);
        break;
      }
      base += total;
    }
  }
  if (s < 0) return;
  const int q0 = p.cu_q[s], ql = p.cu_q[s + 1] - q0;
  const int row_base = b * ROWS;
  const int tok_lo = row_base / Gq, tok_hi = min(ql - 1, (row_base + ROWS - 1) / Gq);
  const int pos_lo = p.positions[q0 + tok_lo], pos_hi = p.positions[q0 + tok_hi];
  const int key_lo = first_key(pos_lo, p.window, p.chunk);
  // key tiles: those of the kept first keys that the window's walk does not reach, [0, n_kept), then the window's,
  // [win0, pos_hi / KEYS]; walked as one list of `n1 - n0` entries
  const int win0 = key_lo / KEYS;
  const int n_kept = min((min(p.keep_first, key_lo) + KEYS - 1) / KEYS, win0);
  int n0 = 0, n1 = n_kept + pos_hi / KEYS + 1 - win0;
  if (p.splits > 1) {
    const int per = (n1 + p.splits - 1) / p.splits;
    n0 = z * per;
    n1 = min(n1, n0 + per);
  }
  auto tile_of = [&](int n) { return n < n_kept ? n : win0 + (n - n_kept); };
  const int* bt = p.block_table + (size_t)s * p.bt_stride;

  // zero the tiles once where a head is narrower than DP: the columns beyond kd / vd are never copied into
  if (p.kd < DP)
    for (int i = tid; i < STAGES * KEYS * LD / 8; i += THREADS) reinterpret_cast<uint4*>(Ks)[i] = make_uint4(0, 0, 0, 0);
  if (p.vd < DP)
    for (int i = tid; i < STAGES * KEYS * LD / 8; i += THREADS) reinterpret_cast<uint4*>(Vs)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();

  const int kchunks = p.kd / 8, vchunks = p.vd / 8;
  // two threads a key row, each with every other 16-byte piece of the key and of the value: one page look-up a
  // thread and tile
  const int lk = tid >> 1, lh = tid & 1;
  auto load_tile = [&](int tile, int stage) {
    const int j = tile * KEYS + lk;
    bool ok = (j >= key_lo || j < p.keep_first) && j <= pos_hi;
    const int pi = p.page_shift >= 0 ? j >> p.page_shift : j / p.page_size;
    const int page = ok ? bt[pi] : -1;
    ok = ok && page >= 0;
    const long long slot = ok ? ((long long)page * p.nkv + g) * p.page_size + (j - pi * p.page_size) : 0;
    const bf16* ksrc = p.kcache + slot * p.kd;
    const bf16* vsrc = p.vcache + slot * p.vd;
    bf16* kdst = Ks + (stage * KEYS + lk) * LD;
    bf16* vdst = Vs + (stage * KEYS + lk) * LD;
    for (int part = lh; part < kchunks; part += 2) cp_async16(kdst + part * 8, ksrc + part * 8, ok);
    for (int part = lh; part < vchunks; part += 2) cp_async16(vdst + part * 8, vsrc + part * 8, ok);
  };

  // this thread's two rows
  constexpr int NT = FEW ? 2 : KEYS / 8;           // tiles of 8 keys a warp takes of a tile of 64
  const int kofs = FEW ? warp * 16 : 0;            // the first of them
  const int r0 = row_base + (FEW ? 0 : warp * 16) + (lane >> 2), r1 = r0 + 8;
  const int t0l = r0 / Gq, t1l = r1 / Gq;
  const bool v0 = t0l < ql, v1 = t1l < ql;
  const int h0 = g * Gq + r0 % Gq, h1 = g * Gq + r1 % Gq;
  const int pos0 = v0 ? p.positions[q0 + t0l] : -1, pos1 = v1 ? p.positions[q0 + t1l] : -1;
  const int st0 = v0 ? first_key(pos0, p.window, p.chunk) : 0, st1 = v1 ? first_key(pos1, p.window, p.chunk) : 0;

  // query fragments (A operand), zero beyond kd and for rows that do not exist
  uint32_t qf[DP / 16][4];
  {
    const bf16* q0p = p.q + (size_t)(q0 + (v0 ? t0l : 0)) * p.q_stride + (size_t)h0 * p.kd;
    const bf16* q1p = p.q + (size_t)(q0 + (v1 ? t1l : 0)) * p.q_stride + (size_t)h1 * p.kd;
#pragma unroll
    for (int ks = 0; ks < DP / 16; ++ks) {
      const int c = ks * 16 + (lane & 3) * 2;
      qf[ks][0] = (v0 && c < p.kd) ? *reinterpret_cast<const uint32_t*>(q0p + c) : 0u;
      qf[ks][1] = (v1 && c < p.kd) ? *reinterpret_cast<const uint32_t*>(q1p + c) : 0u;
      qf[ks][2] = (v0 && c + 8 < p.kd) ? *reinterpret_cast<const uint32_t*>(q0p + c + 8) : 0u;
      qf[ks][3] = (v1 && c + 8 < p.kd) ? *reinterpret_cast<const uint32_t*>(q1p + c + 8) : 0u;
    }
  }

  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const bool first_part = z == 0 && (!FEW || warp == 0);      // the part that opens the softmax (SIG: that owns the 1)
  const bool with_sink = !SIG && p.sinks && first_part;
  float m0 = (with_sink && v0) ? p.sinks[h0] * 1.4426950408889634f : -INFINITY;
  float m1 = (with_sink && v1) ? p.sinks[h1] * 1.4426950408889634f : -INFINITY;
  float l0 = ((with_sink || (SIG && first_part)) && v0) ? 1.f : 0.f, l1 = ((with_sink || (SIG && first_part)) && v1) ? 1.f : 0.f;
  float sb0 = 0.f, sb1 = 0.f;                       // SIG: the heads' biases in the log2 domain
  if (SIG) {
    sb0 = (p.sinks && v0) ? p.sinks[h0] * 1.4426950408889634f : 0.f;
    sb1 = (p.sinks && v1) ? p.sinks[h1] * 1.4426950408889634f : 0.f;
    m0 = v0 ? 0.f : -INFINITY;
    m1 = v1 ? 0.f : -INFINITY;
  }

  // STAGES - 1 tiles are on their way while one is worked on (a commit per tile, empty past the end, so that
  // the count of groups in flight says which tile has landed)
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (n0 + i < n1) load_tile(tile_of(n0 + i), i);
    cp_async_commit();
  }
  for (int n = n0; n < n1; ++n) {
    const int tile = tile_of(n);
    const int stage = (n - n0) % STAGES;
    if (n + STAGES - 1 < n1) load_tile(tile_of(n + STAGES - 1), (n - n0 + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const bf16* kt = Ks + stage * KEYS * LD;
    const bf16* vt = Vs + stage * KEYS * LD;

    float sc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
    // one ldmatrix brings the key fragments of two tiles of 8 keys for 16 dimensions
    const bf16* kr = kt + (kofs + (lane & 7) + (lane >> 4) * 8) * LD + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
#pragma unroll
      for (int ks = 0; ks < DP / 16; ++ks) {
        if (ks * 16 < p.kd) {
          uint32_t kb[4];
          ldmatrix_x4(kb, kr + np * 16 * LD + ks * 16);
          mma_bf16(sc[2 * np], qf[ks], kb[0], kb[1]);
          mma_bf16(sc[2 * np + 1], qf[ks], kb[2], kb[3]);
        }
      }
    }
    // mask (only where a row's edge crosses the tile), scale into the log2 domain, running maximum
    const int key0 = tile * KEYS + kofs;
    float mx0 = -INFINITY, mx1 = -INFINITY;
    const bool edge = !v0 || !v1 || (key0 < max(st0, st1) && key0 + NT * 8 > p.keep_first) ||
                      key0 + NT * 8 - 1 > min(pos0, pos1);
    if (__any_sync(0xffffffffu, edge)) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = key0 + nt * 8 + (lane & 3) * 2 + e;
          const float a = (v0 && (j >= st0 || j < p.keep_first) && j <= pos0) ? sc[nt][e] * p.scale_log2 : -INFINITY;
          const float c = (v1 && (j >= st1 || j < p.keep_first) && j <= pos1) ? sc[nt][2 + e] * p.scale_log2 : -INFINITY;
          sc[nt][e] = a; sc[nt][2 + e] = c;
          mx0 = fmaxf(mx0, a); mx1 = fmaxf(mx1, c);
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nt][e] *= p.scale_log2;
        mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1])); mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
      }
    }
    if (SIG) {
      // sigmoid(x) = 1 / (1 + 2^(-x log2 e)); a masked key's -inf gives 1 / (1 + inf) = 0
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        sc[nt][0] = fast_rcp(1.f + fast_exp2(-(sc[nt][0] + sb0))); sc[nt][1] = fast_rcp(1.f + fast_exp2(-(sc[nt][1] + sb0)));
        sc[nt][2] = fast_rcp(1.f + fast_exp2(-(sc[nt][2] + sb1))); sc[nt][3] = fast_rcp(1.f + fast_exp2(-(sc[nt][3] + sb1)));
      }
    } else {
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
    const float u0 = nm0 == -INFINITY ? 0.f : nm0, u1 = nm1 == -INFINITY ? 0.f : nm1;     // a row that has seen nothing yet
    const float c0 = fast_exp2(m0 - u0), c1 = fast_exp2(m1 - u1);
    m0 = nm0; m1 = nm1;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      sc[nt][0] = fast_exp2(sc[nt][0] - u0); sc[nt][1] = fast_exp2(sc[nt][1] - u0);
      sc[nt][2] = fast_exp2(sc[nt][2] - u1); sc[nt][3] = fast_exp2(sc[nt][3] - u1);
      s0 += sc[nt][0] + sc[nt][1]; s1 += sc[nt][2] + sc[nt][3];
    }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    l0 = l0 * c0 + s0; l1 = l1 * c1 + s1;
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
      pa[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
      pa[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
      pa[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
      const bf16* vr = vt + (kofs + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8;
#pragma unroll
      for (int np = 0; np < DP / 16; ++np) {
        if (np * 16 < p.vd) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vr + np * 16);
          mma_bf16(o[2 * np], pa, vb[0], vb[1]);
          mma_bf16(o[2 * np + 1], pa, vb[2], vb[3]);
        }
      }
    }
    __syncthreads();          // the stage is free for the next iteration's copy
  }
  cp_async_wait<0>();

  if (FEW) {
    // join the four warps' parts in warp order: warp w leaves its rows' sums, maxima and denominators in shared
    // memory (the tiles are done with), then every warp takes a quarter of the columns' work
    __syncthreads();
    float* po = reinterpret_cast<float*>(smem_raw);          // [4][16][DP]
    float* pm = po + 4 * 16 * DP;                            // [4][16], then the denominators [4][16]
    float* pl = pm + 4 * 16;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = (lane >> 2) + half * 8;
#pragma unroll
      for (int i = 0; i < DP / 8; ++i)
        *reinterpret_cast<float2*>(po + (warp * 16 + r) * DP + i * 8 + (lane & 3) * 2) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
      if ((lane & 3) == 0) { pm[warp * 16 + r] = half ? m1 : m0; pl[warp * 16 + r] = half ? l1 : l0; }
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * (p.vd / 2); idx += THREADS) {
      const int r = idx / (p.vd / 2), c = (idx % (p.vd / 2)) * 2;
      const int row = row_base + r, tl = row / Gq;
      if (tl >= ql) continue;
      const int h = g * Gq + row % Gq, t = q0 + tl;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, pm[w * 16 + r]);
      float L = 0.f, a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        if (pm[w * 16 + r] == -INFINITY) continue;
        const float f = fast_exp2(pm[w * 16 + r] - M);
        L = fmaf(pl[w * 16 + r], f, L);
        const float2 ov = *reinterpret_cast<const float2*>(po + (w * 16 + r) * DP + c);
        a0 = fmaf(ov.x, f, a0); a1 = fmaf(ov.y, f, a1);
      }
      if (p.splits > 1) {
        const size_t prow = ((size_t)t * p.nh + h) * p.splits + z;
        *reinterpret_cast<float2*>(p.pacc + prow * p.vd + c) = make_float2(a0, a1);
        if (c == 0) { p.pml[prow * 2] = M; p.pml[prow * 2 + 1] = L; }
      } else {
        float f = L > 0.f ? 1.f / L : 0.f;
        if (p.gate) f *= 1.f / (1.f + __expf(-p.gate[(size_t)t * p.gate_ld + h]));
        *reinterpret_cast<__nv_bfloat162*>(p.out + (size_t)t * p.out_stride + (size_t)h * p.vd + c) = __floats2bfloat162_rn(a0 * f, a1 * f);
      }
    }
    return;
  }

  if (p.splits > 1) {
    // unnormalised parts: [row = token * nh + head][split][vd], and (maximum, denominator)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const bool v = half ? v1 : v0;
      if (!v) continue;
      const size_t row = (size_t)(q0 + (half ? t1l : t0l)) * p.nh + (half ? h1 : h0);
      float* pa = p.pacc + (row * p.splits + z) * p.vd;
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        const int c = i * 8 + (lane & 3) * 2;
        if (c < p.vd) *reinterpret_cast<float2*>(pa + c) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
      }
      if ((lane & 3) == 0) {
        float* ml = p.pml + (row * p.splits + z) * 2;
        ml[0] = half ? m1 : m0;
        ml[1] = half ? l1 : l0;
      }
    }
    return;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const bool v = half ? v1 : v0;
    if (!v) continue;
    const int t = q0 + (half ? t1l : t0l), h = half ? h1 : h0;
    const float l = half ? l1 : l0;
    float f = l > 0.f ? 1.f / l : 0.f;
    if (p.gate) f *= 1.f / (1.f + __expf(-p.gate[(size_t)t * p.gate_ld + h]));
    bf16* op = p.out + (size_t)t * p.out_stride + (size_t)h * p.vd;
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      const int c = i * 8 + (lane & 3) * 2;
      if (c < p.vd) *reinterpret_cast<__nv_bfloat162*>(op + c) = __floats2bfloat162_rn(o[i][half * 2] * f, o[i][half * 2 + 1] * f);
    }
  }
}

// One warp per (token, head): the parts of the key ranges, joined in range order.
__global__ void __launch_bounds__(128) sink_attention_merge_kernel(const float* __restrict__ pacc, const float* __restrict__ pml,
                                                                   bf16* __restrict__ out, long long out_stride, int n_rows,
                                                                   int nh, int vd, int splits, const float* __restrict__ gate,
                                                                   int gate_ld) {
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 4 + warp;
  if (row >= n_rows) return;
  const int t = (int)(row / nh), h = (int)(row % nh);
  const float* ml = pml + (size_t)row * splits * 2;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, ml[2 * s]);
  float L = 0.f;
  for (int s = 0; s < splits; ++s) L += ml[2 * s] == -INFINITY ? 0.f : ml[2 * s + 1] * exp2f(ml[2 * s] - M);
  float f = L > 0.f ? 1.f / L : 0.f;
  if (gate) f *= 1.f / (1.f + __expf(-gate[(size_t)t * gate_ld + h]));
  for (int c = lane; c < vd; c += 32) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s)
      if (ml[2 * s] != -INFINITY) a = fmaf(pacc[((size_t)row * splits + s) * vd + c], exp2f(ml[2 * s] - M), a);
    out[(size_t)t * out_stride + (size_t)h * vd + c] = __float2bfloat16_rn(a * f);
  }
}

}  // namespace sinkmma

RLLM_API int rllm_sink_attention_mma_supported(int dt, int kd, int vd, int page_size) {
  return dt == DT_BF16 && kd > 0 && vd > 0 && kd % 16 == 0 && vd % 16 == 0 && kd <= 128 && vd <= 128 && page_size > 0;
}

// As rllm_sink_attention_simt, bfloat16 only. cu_q [num_seqs + 1]: the row range of each sequence (rows of a
// sequence adjacent, positions ascending). splits > 1: pacc float [n_tokens * nh, splits, vd], pml float [.., splits, 2].
RLLM_API int rllm_sink_attention_mma(const void* q, long long q_stride, const void* kcache, const void* vcache, void* out,
                                     long long out_stride, const int* positions, const int* cu_q, const int* block_table,
                                     int bt_stride, int num_seqs, int n_tokens, int max_q_len, int nh, int nkv, int kd, int vd,
                                     int page_size, float scale, int window, int chunk, const float* sinks, const float* gate,
                                     int gate_ld, int splits, float* pacc, float* pml, int keep_first, int sigmoid,
                                     void* stream) {
  using namespace sinkmma;
  if (n_tokens <= 0 || num_seqs <= 0) return 0;
  if (!rllm_sink_attention_mma_supported(DT_BF16, kd, vd, page_size) || nkv <= 0 || nh % nkv || splits < 1 || splits > 64 ||
      keep_first < 0)
    return ERR_BAD_SIZE;
  if (q_stride % 2 || out_stride % 2 || (splits > 1 && (!pacc || !pml))) return ERR_BAD_ALIGN;
  const int Gq = nh / nkv;
  const long long tiles = ((long long)n_tokens * Gq + ROWS - 1) / ROWS + num_seqs;
  if (tiles > 2147483647LL || nkv > 65535) return ERR_TOO_LARGE;
  Args a = {(const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache, (bf16*)out, out_stride, positions, cu_q,
            block_table, bt_stride, num_seqs, nh, nkv, kd, vd, page_size, scale * 1.4426950408889634f, window, chunk, sinks,
            gate, gate_ld, splits, pacc, pml, -1, keep_first};
  for (int sft = 0; sft < 31; ++sft) if ((1 << sft) == page_size) a.page_shift = sft;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid((unsigned)tiles, (unsigned)nkv, (unsigned)splits);
  const int dp = (kd <= 64 && vd <= 64) ? 64 : 128;
  const int smem = 2 * STAGES * KEYS * (dp + 8) * (int)sizeof(bf16);     // also holds the FEW join: 4 x 16 x (dp + 2) floats
  const bool few = (long long)max_q_len * Gq <= 16;             // every sequence's rows fit one warp's 16
  int rc;
#define GO(D, F, G)                                                                                     \
  {                                                                                                     \
    static bool done[64] = {};                                                                          \
    if ((rc = allow_dynamic_smem(sink_attention_mma_kernel<D, F, G>, smem, done))) return rc;           \
    rc = launch_ex(sink_attention_mma_kernel<D, F, G>, grid, dim3(THREADS), (size_t)smem, s, 1, a);     \
  }
#define GO2(D, F) { if (sigmoid) GO(D, F, true) else GO(D, F, false) }
  if (dp == 64) { if (few) GO2(64, true) else GO2(64, false) }
  else { if (few) GO2(128, true) else GO2(128, false) }
#undef GO2
#undef GO
  if (rc || splits == 1) return rc;
  const long long rows = (long long)n_tokens * nh;
  return launch_ex(sink_attention_merge_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, s, 1, (const float*)pacc,
                   (const float*)pml, (bf16*)out, out_stride, (int)rows, nh, vd, splits, gate, gate_ld);
}
