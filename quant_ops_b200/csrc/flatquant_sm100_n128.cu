// FlatQuant quantizer for sm_100a, right transform of size 80, 96, 112 or 128 (features = M x N, 16 <= M <= 128): the
// hidden sizes 14336 = 112 x 128, 11008 = 86 x 128, 8192 = 64 x 128, 7168 = 64 x 112, 6144 = 64 x 96, 5120 = 64 x 80
// run here.  For N < 128 everything is laid out as for N = 128: the TMA fills the missing columns of X with zeros,
// R is staged with zero columns, so the extra columns of Y and Z are exact zeros; they are not stored.
//
// One persistent CTA per SM works on tiles of G tokens: G = 2 when M <= 64 and M is a multiple of 16, else G = 1.
//
//   warp 0       TMA: 3-D tensor map (n, m, token), two boxes of 64 x M x G per tile (the two 64-column halves of the
//                rows), 128-byte swizzle, 2 stages
//   warp 1       issues Y = X . R        A = X rows (K-major), B = R as it lies in memory (N-major), M = 128, N = 128,
//                                        K = 128
//   warp 2       issues Z = LL . Y       A = LL: L^T in rows 0 .. M-1, and for G = 2 a second copy below it, staged as
//                                        the rows of L laid along M (M-major): neither transform is transposed;
//                                        B = Y (N-major).  G = 1: N = 128.  G = 2: one MMA of N = 256 per K step, the
//                                        64-column blocks of both tokens interleaved along N, K = M
//   warps 3-10   Y pass: tensor memory -> round to the activation dtype -> shared memory in the B layout;
//                warp (q, h) handles columns 64h .. 64h+63 of tensor-memory lanes 32q .. 32q+31
//   warps 11-26  quantize pass, 16 warps: warp (q, h) handles columns 32h .. 32h+31 of lanes 32q .. 32q+31; a thread
//                rounds its 32 values once (packed pairs), the token's absmax is combined through shared memory, then
//                scale, int4 codes and one 16-byte store.  The Z accumulators are released as soon as they sit in
//                registers, so the next tile's second product overlaps with the arithmetic.
//
// With the stacked copy of L^T, lane block c holds the Z rows of token c, as in flatquant_sm100_n64.cu, whose packed
// arithmetic (flatquant_sm100_common.cuh) this kernel shares.  Rows of a tile that only pad the reduction length of
// the second product (M not a multiple of 16) are written as exact zeros by the Y pass.
//
// Rounding points and the exactness arguments are those of flatquant_sm100.cu (reference:
// src/quant_ops/ops/quantization/flatquant/ops.py:99-117).  Every mbarrier wait is bounded.
#include "flatquant_sm100_common.cuh"

namespace qo {
namespace {

using namespace ptx;
using namespace fq;

constexpr int kThreads = 864;                  // 27 warps: TMA, two MMA issuers, 8 (Y pass) + 16 (quantize pass)
constexpr int kEpi1Warp0 = 3, kEpi2Warp0 = 11;
constexpr int kXStages = 2, kYStages = 2;      // kYStages also counts the Y accumulator stages
constexpr int kStageBytes = 2 * kAtomBytes;    // 128 rows x 256 bytes, as two 64-column atoms
constexpr int kOffX = 0;
constexpr int kOffY = kOffX + kXStages * kStageBytes;
constexpr int kOffR = kOffY + kYStages * kStageBytes;
constexpr int kOffLL = kOffR + 2 * kAtomBytes;
constexpr int kOffMisc = kOffLL + 2 * kAtomBytes;
constexpr int kSmemBytes = kOffMisc + 1024 + 1024;
constexpr int kTmemCols = 512;                 // Y accumulators: 2 stages x 128 columns; Z accumulators: 256 columns
constexpr int kColZ = 256;

struct Misc {
  uint64_t full_x[kXStages], empty_x[kXStages];
  uint64_t d1_full[kYStages], d1_empty[kYStages], y_full[kYStages], y_empty[kYStages];
  uint64_t d2_full[2], d2_empty[2], set_sync;
  uint32_t tmem_base;
  int absmax_bits[3][2];
};

// FULL: the right transform is 128 wide (compile-time widths keep the common shapes free of the narrow-case tests)
template <typename T, int MODE, bool FULL>
__global__ void __launch_bounds__(kThreads, 1)
flatquant_n128_kernel(const __grid_constant__ CUtensorMap x_map, const T* __restrict__ left, const T* __restrict__ right,
                      void* __restrict__ out, void* __restrict__ scales, long long tokens, int m, int nc_arg, int group, float clip,
                      int scale_dtype, uint32_t* __restrict__ status) {
  const int nc = FULL ? 128 : nc_arg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + kOffMisc);
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rows_tile = group * m;            // X / Y rows per tile (<= 128)
  const int k2 = (m + 15) & ~15;              // reduction length of the second product
  const int y_atom = group == 2 ? 2 * m * 128 : kAtomBytes;  // bytes between the two 64-column halves of a Y stage
  const long long ntiles = (tokens + group - 1) / group;
  // Warps whose 32 tensor-memory lanes carry no row of the tile take no part: they skip their role and the barrier
  // counts below only include the others (M = 86: the fourth quadrant of both passes is idle).
  const int mpad32 = (m + 31) & ~31;
  const int nq1 = ((group == 1 ? k2 : rows_tile) + 31) >> 5;  // quadrants with rows in the Y pass
  int nq2 = 0;                                                // quadrants with rows in the quantize pass
  for (int qq = 0; qq < 4; ++qq) {
    const int cc = (qq * 32) / mpad32;
    nq2 += (cc < group && qq * 32 - cc * mpad32 < m) ? 1 : 0;
  }
  const int nh2 = (nc + 31) >> 5;             // 32-column blocks of Z that hold real columns (quantize-pass warps per quadrant)
  int mine = 0;                               // tiles this CTA works on
  if ((long long)blockIdx.x < ntiles) mine = (int)((ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x);

  if (tid == 0) {
    for (int i = 0; i < kXStages; ++i) { mbar_init(smem_u32(&misc->full_x[i]), 1); mbar_init(smem_u32(&misc->empty_x[i]), 1); }
    for (int i = 0; i < kYStages; ++i) {
      mbar_init(smem_u32(&misc->d1_full[i]), 1);
      mbar_init(smem_u32(&misc->d1_empty[i]), 2 * nq1);  // one arrival per working warp of the Y pass
      mbar_init(smem_u32(&misc->y_full[i]), 2 * nq1);
      mbar_init(smem_u32(&misc->y_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&misc->d2_full[i]), 1);
      mbar_init(smem_u32(&misc->d2_empty[i]), nh2 * nq2);  // one arrival per working warp of the quantize pass
    }
    mbar_init(smem_u32(&misc->set_sync), nh2 * nq2);
    for (int i = 0; i < 3 * 2; ++i) (&misc->absmax_bits[0][0])[i] = 0;
    fence_barrier_init();
    prefetch_tensormap(&x_map);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&misc->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();  // barriers and the tensor-memory base exist; the producer starts filling the X stages
  tc_fence_after();
  const uint32_t tmem = misc->tmem_base;
  // Programmatic dependent launch: everything above overlaps with the tail of the preceding kernel of the stream;
  // nothing below (reads of X, L, R, writes of the outputs) starts before that kernel has completed.
  grid_dependency_wait();
  // Only now may a dependent launch start early: whatever it reads before its own wait (a following GEMM prefetches
  // its weights) was then written by kernels that completed before this one passed the wait above.
  grid_launch_dependents();

  if (warp != 0) {
    // Both transforms are staged as they lie in memory, 16 bytes at a time with the 128-byte XOR swizzle: the tensor
    // core reads R as an N-major B operand (row k of R = 128-byte rows of the two 64-column blocks) and L as an
    // M-major A operand (row k of L laid along M, once per token copy), so nothing is transposed here.
    constexpr int kStagers = kThreads - 32;
    const int t13 = tid - 32;
    // Every thread first requests all its pieces of both transforms (at most three each) and only then stores them: the
    // loads come from L2 with several hundred cycles of latency each, and this staging is on the path of the first tile.
    // R: rows k < nc, 16 pieces per row; columns past nc are zero (the first product always has N = 128)
    // LL: rows k < k2 (rows m .. k2-1 pad the reduction length and must be zero), M position copy * mpad + i holds
    // L[k][i]; every other M position of these rows is zero
    static_assert(3 * kStagers >= 128 * 16, "three pieces per thread cover a transform");
    const int mpad = (m + 31) & ~31;  // the second copy starts on a 32-row boundary: a warp reads one token's columns
    const bool l_vec = (m & 7) == 0;  // rows of L start on 16-byte boundaries
    uint4 wr[3], wl[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int idx = t13 + j * kStagers, k = idx >> 4, c = idx & 15;
      wr[j] = make_uint4(0, 0, 0, 0);
      if (idx < nc * 16 && 8 * c < nc) wr[j] = *reinterpret_cast<const uint4*>(right + k * nc + 8 * c);
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int idx = t13 + j * kStagers, k = idx >> 4, c = idx & 15;
      const int cpy = (8 * c) / mpad, i0 = 8 * c - cpy * mpad;
      wl[j] = make_uint4(0, 0, 0, 0);
      if (idx < k2 * 16 && k < m && cpy < group && i0 < m) {
        const T* src = left + k * m + i0;
        if (l_vec) {
          wl[j] = *reinterpret_cast<const uint4*>(src);
        } else {
          uint32_t e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) e[i] = i0 + i < m ? (uint32_t)reinterpret_cast<const uint16_t*>(src)[i] : 0u;
          wl[j] = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int idx = t13 + j * kStagers, k = idx >> 4, c = idx & 15;
      if (idx < nc * 16) *reinterpret_cast<uint4*>(smem + kOffR + (c >> 3) * kAtomBytes + k * 128 + (((c & 7) ^ (k & 7)) << 4)) = wr[j];
      if (idx < k2 * 16) *reinterpret_cast<uint4*>(smem + kOffLL + (c >> 3) * kAtomBytes + k * 128 + (((c & 7) ^ (k & 7)) << 4)) = wl[j];
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, %0;" ::"n"(kStagers) : "memory");
  }

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t bytes = (uint32_t)(rows_tile * 256);
      int s = 0, ph = 0;
      long long tile = blockIdx.x;
      for (int it = 0; it < mine; ++it, tile += gridDim.x) {
        if (!mbar_wait(smem_u32(&misc->empty_x[s]), ph ^ 1)) { atomicCAS(status, 0u, 0x900u + s); break; }
        const uint32_t bar = smem_u32(&misc->full_x[s]);
        mbar_arrive_expect_tx(bar, bytes);
        tma_load_3d(smem_base + kOffX + s * kStageBytes, &x_map, bar, 0, 0, (int)(tile * group));
        tma_load_3d(smem_base + kOffX + s * kStageBytes + kAtomBytes, &x_map, bar, 64, 0, (int)(tile * group));
        if (++s == kXStages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc1 = umma_idesc(1, Fmt<T>::id, Fmt<T>::id, 0, 1, 128, 128);  // B = R as it lies in memory: N-major
      const uint64_t desc_x0 = umma_smem_desc_sw128(smem_base + kOffX, 16, 1024);
      const uint64_t desc_r = umma_smem_desc_sw128(smem_base + kOffR, kAtomBytes, 1024);  // 64-column blocks one atom apart
      int sx = 0, phx = 0, s1 = 0, ph1 = 0;
      for (int it = 0; it < mine; ++it) {
        if (const int w = mbar_wait2(smem_u32(&misc->full_x[sx]), phx, smem_u32(&misc->d1_empty[s1]), ph1 ^ 1)) {
          atomicCAS(status, 0u, 0x900u + 0x10u * w + sx);
          break;
        }
        tc_fence_after();
        const uint64_t da = desc_x0 + (uint64_t)(sx * (kStageBytes >> 4));
        if (FULL) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t off = (uint64_t)((ks >> 2) * (kAtomBytes >> 4) + (ks & 3) * 2);  // K atom, then 32 bytes per step
            mma_f16_ss(tmem + s1 * 128, da + off, desc_r + (uint64_t)(ks * 128), idesc1, ks);  // 16 rows of R = 2048 bytes per step
          }
        } else {
#pragma unroll 1
          for (int ks = 0; ks < (nc >> 4); ++ks) {
            const uint64_t off = (uint64_t)((ks >> 2) * (kAtomBytes >> 4) + (ks & 3) * 2);
            mma_f16_ss(tmem + s1 * 128, da + off, desc_r + (uint64_t)(ks * 128), idesc1, ks);
          }
        }
        mma_commit(smem_u32(&misc->empty_x[sx]));
        mma_commit(smem_u32(&misc->d1_full[s1]));
        if (++sx == kXStages) { sx = 0; phx ^= 1; }
        if (++s1 == kYStages) { s1 = 0; ph1 ^= 1; }
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {
      const uint32_t idesc2 = umma_idesc(1, Fmt<T>::id, Fmt<T>::id, 1, 1, 128, group == 2 ? 256 : nc);  // A = LL, M-major
      const uint64_t desc_ll = umma_smem_desc_sw128(smem_base + kOffLL, kAtomBytes, 1024);  // 64-row blocks one atom apart
      // N-major B operand: the stride between 64-column blocks along N is m rows (G = 2: token blocks interleave
      // with the column halves) or one atom (G = 1)
      const uint64_t desc_y0 = umma_smem_desc_sw128(smem_base + kOffY, group == 2 ? (uint32_t)(m * 128) : (uint32_t)kAtomBytes, 1024);
      const int ksteps2 = k2 >> 4;
      int sy = 0, phy = 0;
      for (int it = 0; it < mine; ++it) {
        const int e = group == 2 ? 0 : (it & 1), ph = (group == 2 ? it : (it >> 1)) & 1;
        if (const int w = mbar_wait2(smem_u32(&misc->y_full[sy]), phy, smem_u32(&misc->d2_empty[e]), ph ^ 1)) {
          atomicCAS(status, 0u, 0x920u + 0x10u * w + sy);
          break;
        }
        tc_fence_after();
        const uint64_t db0 = desc_y0 + (uint64_t)(sy * (kStageBytes >> 4));
#pragma unroll 1
        for (int ks = 0; ks < ksteps2; ++ks) {
          const uint64_t da2 = desc_ll + (uint64_t)(ks * 128);  // 16 rows of L = 2048 bytes per step
          mma_f16_ss(tmem + kColZ + e * 128, da2, db0 + (uint64_t)(ks * 128), idesc2, ks);  // 16 Y rows = 2048 bytes per step
        }
        mma_commit(smem_u32(&misc->y_empty[sy]));
        mma_commit(smem_u32(&misc->d2_full[e]));
        if (++sy == kYStages) { sy = 0; phy ^= 1; }
      }
    }
  } else if (warp < kEpi2Warp0) {
    // ---- Y pass: 8 warps; warp (q, h) converts columns 64h .. 64h+63 of tensor-memory lanes 32q .. 32q+31 ------
    const int q = warp & 3, h = (warp - kEpi1Warp0) >> 2, r = q * 32 + lane;
    int s = 0, ph = 0;
    for (int it = 0; it < (q < nq1 ? mine : 0); ++it) {
      if (__any_sync(0xffffffffu, mbar_wait2(smem_u32(&misc->d1_full[s]), ph, smem_u32(&misc->y_empty[s]), ph ^ 1) != 0)) {
        atomicCAS(status, 0u, 0xA00u + s);
        break;
      }
      tc_fence_after();
      // (rows start on 128-byte boundaries: piece c of the swizzled row is at (row | (r & 7) << 4) ^ (c << 4), one logic
      // operation per store instead of three)
      const uint32_t yrow = (smem_base + kOffY + s * kStageBytes + h * y_atom + r * 128) | (uint32_t)((r & 7) << 4);
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + s * 128 + h * 64 + p * 32, v);
        tmem_ld_wait();
        if (p == 1) {
          tc_fence_before();
          mbar_arrive_warp(smem_u32(&misc->d1_empty[s]));  // accumulators are in registers: the stage can be overwritten
        }
        if (r < rows_tile || (group == 1 && r < k2)) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w = make_uint4(0, 0, 0, 0);  // rows that only pad the reduction length must be exact zeros
            if (r < rows_tile) {
              w.x = pack2<T>(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
              w.y = pack2<T>(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              w.z = pack2<T>(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              w.w = pack2<T>(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            }
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(yrow ^ (uint32_t)((p * 4 + j) << 4)), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
          }
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(smem_u32(&misc->y_full[s]));
      if (++s == kYStages) { s = 0; ph ^= 1; }
    }
  } else {
    // ---- quantize pass: 16 warps; warp (q, h) works on columns 32h .. 32h+31 of lanes 32q .. 32q+31 -----------
    const int q = warp & 3, h = (warp - kEpi2Warp0) >> 2, l = q * 32 + lane;
    const int mpad = (m + 31) & ~31;
    const int c = l / mpad, mi = l - c * mpad;  // lane block c holds the Z rows of token c (copies start on warp boundaries)
    const bool active = c < group && mi < m;
    constexpr bool warp_uniform = true;         // all rows of a warp belong to one token
    const int feat = m * nc;
    const int c0 = h * 32;
    const int cols = FULL ? 32 : min(32, max(0, nc - c0));  // real columns among this warp's 32 (a multiple of 16)
    // G = 1: two accumulator stages of 128 columns, natural column order.  G = 2: one stage of 256 columns whose
    // 64-column blocks are ordered (half 0, token 0), (half 0, token 1), (half 1, token 0), (half 1, token 1).
    const uint32_t col_in_stage = group == 2 ? (uint32_t)((((h >> 1) * 2 + (active ? c : 0)) * 64) + (h & 1) * 32) : (uint32_t)c0;
    long long tile = blockIdx.x;
    const bool warp_works = (q * 32) / mpad < group && q * 32 - ((q * 32) / mpad) * mpad < m && cols > 0;
    for (int it = 0; it < (warp_works ? mine : 0); ++it, tile += gridDim.x) {
      const int e = group == 2 ? 0 : (it & 1), use = group == 2 ? it : (it >> 1);
      const int buf = it % 3;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&misc->d2_full[e]), use & 1))) { atomicCAS(status, 0u, 0xB00u + e); break; }
      tc_fence_after();
      const long long tok = tile * group + c;
      const bool valid = active && tok < tokens;
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + kColZ + e * 128 + col_in_stage, v);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(smem_u32(&misc->d2_empty[e]));  // the Z accumulators of this stage are free again
      if (cols < 32) {
        // N = 80 or 112: the upper 16 columns of this block were not written by the second product (its N is the
        // real width when a tile is one token); they must not reach the absmax
#pragma unroll
        for (int j = 16; j < 32; ++j) v[j] = 0u;
      }

      if (MODE == kTransform) {
        if (valid) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + tok * feat + mi * nc + c0);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (4 * j < cols) dst[j] = make_float4(DT<T>::rnd(__uint_as_float(v[4 * j])), DT<T>::rnd(__uint_as_float(v[4 * j + 1])),
                                 DT<T>::rnd(__uint_as_float(v[4 * j + 2])), DT<T>::rnd(__uint_as_float(v[4 * j + 3])));
        }
        continue;
      }

      // round Z to the activation dtype once, as packed pairs; both passes work on the pairs
      uint32_t zz[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) zz[i] = P2<T>::cvt(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
      uint32_t m0 = zz[0], m1 = zz[1], m2 = zz[2], m3 = zz[3];  // four chains keep the dependent latency short
#pragma unroll
      for (int i = 4; i < 16; i += 4) {
        m0 = P2<T>::absmax(m0, zz[i]);
        m1 = P2<T>::absmax(m1, zz[i + 1]);
        m2 = P2<T>::absmax(m2, zz[i + 2]);
        m3 = P2<T>::absmax(m3, zz[i + 3]);
      }
      m0 = P2<T>::absmax(P2<T>::absmax(m0, m1), P2<T>::absmax(m2, m3));
      float amax = valid ? fmaxf(fabsf(P2<T>::lo(m0)), fabsf(P2<T>::hi(m0))) : 0.f;
      const float row_amax = amax;  // this row's own extreme, used below to skip the clamp
      if (warp_uniform) {
        amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));  // non-negative floats order as integers
        if (lane == 0 && active) atomicMax(&misc->absmax_bits[buf][c], __float_as_int(amax));
      } else if (active) {
        atomicMax(&misc->absmax_bits[buf][c], __float_as_int(amax));
      }
      // the 16 warps meet here (bounded); afterwards the slot holds the token's absmax
      const uint32_t gs = smem_u32(&misc->set_sync);
      mbar_arrive_warp(gs);
      if (!__all_sync(0xffffffffu, mbar_wait(gs, it & 1))) { atomicCAS(status, 0u, 0xB10u); break; }
      if (active) amax = __int_as_float(misc->absmax_bits[buf][c]);
      if (h == 0 && l < 2) misc->absmax_bits[(it + 2) % 3][l] = 0;
      // max of the rounded values = rounded max; clip * absmax and the division by 7 are rounded like the reference.
      // top / 7 can neither hit nor come within 2^-13 (relative) of a midpoint of the 16-bit format, so the
      // float32 product with 1/7 rounds to the same 16-bit value as the exact quotient.
      const float top = rnd1<T>(amax * clip);  // amax already is a value of the activation dtype
      const float s = fmaxf(rnd1<T>(top * 0.142857149f), DT<T>::floor_scale());
      const float inv_s = __frcp_rn(s);
      uint32_t rhi2, rlo2;  // 1/s as two packed terms of the activation dtype (bf16 only)
      P2<T>::recip2(inv_s, rhi2, rlo2);
      if (valid && mi == 0 && h == 0) store_scale(scales, tok, s, scale_dtype);
      // a quotient can only leave [-8, 7] after rounding if some |z| / s reaches 7.5; most warps have no such row
      const bool clamp_needed = __any_sync(0xffffffffu, !(row_amax * inv_s < 7.4f));
      const bool zero_scale = s == 0.f;

      if (MODE == kPacked && !zero_scale) {
        uint32_t w[4];
        if (clamp_needed) {
#pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = quantize8<T, true>(&zz[4 * j], s, inv_s, rhi2, rlo2);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = quantize8<T, false>(&zz[4 * j], s, inv_s, rhi2, rlo2);
        }
        if (valid) store_words(reinterpret_cast<uint32_t*>(out) + tok * (feat / 8) + (mi * nc + c0) / 8, w, cols);
      } else {
        uint32_t pb[4], qb[4];
        if (!zero_scale) {
#pragma unroll
          for (int j = 0; j < 4; ++j) nibble_bytes_packed<T>(&zz[4 * j], s, inv_s, rhi2, rlo2, pb[j], qb[j]);
        } else {
          // the reference divides by zero here: +-inf clamps to 7 / -8, 0/0 counts as 0
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            pb[j] = qb[j] = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t pz = zz[4 * j + (i >> 1)], qz = zz[4 * j + 2 + (i >> 1)];
              const float z0 = (i & 1) ? P2<T>::hi(pz) : P2<T>::lo(pz), z1 = (i & 1) ? P2<T>::hi(qz) : P2<T>::lo(qz);
              pb[j] |= (uint32_t)(z0 > 0.f ? 15 : (z0 < 0.f ? 0 : 8)) << (8 * i);
              qb[j] |= (uint32_t)(z1 > 0.f ? 15 : (z1 < 0.f ? 0 : 8)) << (8 * i);
            }
          }
        }
        if (MODE == kPacked) {
          if (valid) {
            const uint32_t w[4] = {pack8(pb[0], qb[0]), pack8(pb[1], qb[1]), pack8(pb[2], qb[2]), pack8(pb[3], qb[3])};
            store_words(reinterpret_cast<uint32_t*>(out) + tok * (feat / 8) + (mi * nc + c0) / 8, w, cols);
          }
        } else if (valid) {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<int8_t*>(out) + tok * feat + mi * nc + c0);  // 16-byte aligned: N % 16 == 0
          dst[0] = make_uint4(bytes4(pb[0]), bytes4(qb[0]), bytes4(pb[1]), bytes4(qb[1]));
          if (cols > 16) dst[1] = make_uint4(bytes4(pb[2]), bytes4(qb[2]), bytes4(pb[3]), bytes4(qb[3]));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <typename T, int MODE, bool FULL>
int launch_one(const CUtensorMap& map, const void* left, const void* right, void* out, void* scales, int64_t tokens, int m,
               int nc, float clip, int scale_dtype, uint32_t* status, cudaStream_t stream) {
  auto kern = flatquant_n128_kernel<T, MODE, FULL>;
  int dev = 0, sms = 148;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    QO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[dev & 63] = true;
  }
  sms = sm_count(dev);
  const int group = flatquant_sm100_n128_group(m);
  const int64_t ntiles = (tokens + group - 1) / group;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  QO_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, map, reinterpret_cast<const T*>(left), reinterpret_cast<const T*>(right), out, scales,
                                 (long long)tokens, m, nc, group, clip, scale_dtype, status));
  return check_launch("flatquant_n128_kernel");
}

template <typename T>
int launch_mode(int mode, const CUtensorMap& map, const void* left, const void* right, void* out, void* scales,
                int64_t tokens, int m, int nc, float clip, int scale_dtype, uint32_t* status, cudaStream_t stream) {
  if (nc == 128) {
    switch (mode) {
      case kInt8: return launch_one<T, kInt8, true>(map, left, right, out, scales, tokens, m, nc, clip, scale_dtype, status, stream);
      case kPacked: return launch_one<T, kPacked, true>(map, left, right, out, scales, tokens, m, nc, clip, scale_dtype, status, stream);
      default: return launch_one<T, kTransform, true>(map, left, right, out, scales, tokens, m, nc, clip, scale_dtype, status, stream);
    }
  }
  switch (mode) {
    case kInt8: return launch_one<T, kInt8, false>(map, left, right, out, scales, tokens, m, nc, clip, scale_dtype, status, stream);
    case kPacked: return launch_one<T, kPacked, false>(map, left, right, out, scales, tokens, m, nc, clip, scale_dtype, status, stream);
    default: return launch_one<T, kTransform, false>(map, left, right, out, scales, tokens, m, nc, clip, scale_dtype, status, stream);
  }
}

}  // namespace

bool flatquant_sm100_n128_supported(int m, int n) { return n > 64 && n <= 128 && (n % 16) == 0 && m >= 16 && m <= 128; }
int flatquant_sm100_n128_group(int m) { return (m <= 64 && (m % 16) == 0) ? 2 : 1; }

int launch_flatquant_sm100_n128(int mode, const void* x_map, const void* left, const void* right, void* out, void* scales,
                                int64_t tokens, int m, int n, float clip, int in_dtype, int scale_dtype, uint32_t* status,
                                cudaStream_t stream) {
  const CUtensorMap& map = *reinterpret_cast<const CUtensorMap*>(x_map);
  if (in_dtype == QO_BF16)
    return launch_mode<__nv_bfloat16>(mode, map, left, right, out, scales, tokens, m, n, clip, scale_dtype, status, stream);
  return launch_mode<__half>(mode, map, left, right, out, scales, tokens, m, n, clip, scale_dtype, status, stream);
}

}  // namespace qo
