// FlatQuant quantizer for sm_100a, right transform of size 64 (features = M x 64 with M = 16, 24, ... 64):
// the activation-scale configuration (4096 = 64 x 64) runs here.  Right transforms of 16, 32 and 48 (1024 = 32 x 32,
// 1536 = 32 x 48, 256 = 16 x 16) use the same layout: the TMA fills the missing columns of X with zeros, R is staged
// with zero columns, so the extra columns of Y and Z are exact zeros; they are not stored.
//
// One persistent CTA per SM works on groups of 2 tokens (2M <= 128 rows of 64 elements):
//
//   warp 0       TMA: 3-D tensor map (n, m, token), box 64 x M x 2 -> 2M rows of 128 bytes, 128-byte swizzle, 6 stages
//   warp 1       issues Y = X . R        A = X rows (K-major), B = R as it lies in memory (N-major), M = 128, N = 64,
//                                        K = 64
//   warp 2       issues Z = LL . Y2      A = LL = 2 copies of L^T, each starting on a 32-row boundary; staged as the
//                                        rows of L laid along M (M-major), so neither transform is transposed;
//                                        B = the 2 tokens' Y side by side along N (N-major, N = 128), K = M
//   warps 3-10   Y pass: tensor memory -> round to the activation dtype -> shared memory in the B layout; two sets of
//                four warps that alternate between groups (a group's trip through this pass is a chain of fixed
//                latencies -- barrier poll, tensor-memory load, proxy fence, arrival -- of about the time the rest of
//                the pipeline needs per group; one set working on every group was the kernel's serial bottleneck);
//                warp q of a set handles all 64 columns of tensor-memory lanes 32q..32q+31, 32 at a time
//   warps 11-26  quantize pass, two sets of 8 warps that alternate between groups; lane block c of a set holds a copy
//                of the Z rows and serves token c; a thread rounds its 32 values once (packed pairs), the token's
//                absmax is combined through shared memory, then scale, int4 codes and one 16-byte store
//
// Stacking copies of L^T makes every copy's lanes hold the same Z rows, so different lane blocks can serve
// different tokens and nothing is multiplied by block-diagonal padding.  The accumulator stages are released as
// soon as their values sit in registers.  What the cycle counters showed while shaping this kernel: a try_wait
// costs about 170 cycles even on a completed phase (two barriers are therefore polled together), an mbarrier
// arrival is an atomic on one word (one arrival per warp, not per thread), a tcgen05.mma costs about the same for
// N = 64 as for N = 128, and integer / conversion work runs on the half-rate ALU pipe (the nibble packing uses
// integer multiply-adds instead).
//
// Rounding points and the exactness arguments are those of flatquant_sm100.cu (reference:
// src/quant_ops/ops/quantization/flatquant/ops.py:99-117).  Every mbarrier wait is bounded.
#include "flatquant_sm100_common.cuh"

namespace qo {
namespace {

using namespace ptx;
using namespace fq;

constexpr int kThreads = 864;                  // 27 warps: TMA, two MMA issuers, 8 (Y pass) + 2 x 8 (quantize pass)
constexpr int kEpi1Warp0 = 3, kEpi2Warp0 = 11; // first warp of the Y pass / of the two quantize sets
constexpr int kGroup = 2;                      // tokens per group
constexpr int kXStages = 6;
constexpr int kYStages = 4;                    // also the number of Y accumulator stages; even: each Y-pass set owns two
constexpr int kStageBytes = 128 * 128;         // up to 2 x 64 rows of 128 bytes
constexpr int kOffX = 0;
constexpr int kOffY = kOffX + kXStages * kStageBytes;
constexpr int kOffR = kOffY + kYStages * kStageBytes;
constexpr int kOffLL = kOffR + 64 * 128;
constexpr int kOffMisc = kOffLL + kAtomBytes;
constexpr int kSmemBytes = kOffMisc + 1024 + 1024;
constexpr int kTmemCols = 512;                 // Y accumulators: 4 stages x 64 columns; Z accumulators: 2 stages x 128
constexpr int kColZ = 256;

struct Misc {
  uint64_t full_x[kXStages], empty_x[kXStages];
  uint64_t d1_full[kYStages], d1_empty[kYStages], y_full[kYStages], y_empty[kYStages];
  uint64_t d2_full[2], d2_empty[2], set_sync[2];
  uint32_t tmem_base;
  alignas(16) float absmax_part[2][3][2][4];  // [set][use % 3][token][warp of the token]: per-warp maxima, never-written slots stay 0
};

// FULL: the right transform is 64 wide (compile-time widths keep the benchmarked shape free of the narrow-case tests)
template <typename T, int MODE, bool FULL>
__global__ void __launch_bounds__(kThreads, 1)
flatquant_n64_kernel(const __grid_constant__ CUtensorMap x_map, const T* __restrict__ left, const T* __restrict__ right,
                     void* __restrict__ out, void* __restrict__ scales, long long tokens, int m, int nc_arg, float clip,
                     int scale_dtype, uint32_t* __restrict__ status) {
  const int nc = FULL ? 64 : nc_arg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + kOffMisc);
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mpad = (m + 31) & ~31;            // each copy of L^T starts on a 32-lane boundary: a warp reads one token's columns
  const int rows_group = kGroup * m;          // X rows per group (<= 128)
  const int k2 = (m + 15) & ~15;              // reduction length of the second product; a token's Y rows start at c * k2
  const long long ngroups = (tokens + kGroup - 1) / kGroup;
  // Warps whose 32 tensor-memory lanes carry no row take no part: they skip their role and the barrier counts
  // below only include the others (M = 32: the upper two quadrants of both passes are idle).
  const int nq1 = (rows_group + 31) >> 5;     // quadrants with rows in the Y pass
  int nq2 = 0;                                // quadrants with rows in the quantize pass
  for (int qq = 0; qq < 4; ++qq) {
    const int cc = (qq * 32) / mpad;
    nq2 += (cc < kGroup && qq * 32 - cc * mpad < m) ? 1 : 0;
  }
  const int nh2 = (nc + 31) >> 5;             // 32-column halves of Z that hold real columns
  int mine = 0;                               // groups this CTA works on
  if ((long long)blockIdx.x < ngroups) mine = (int)((ngroups - blockIdx.x + gridDim.x - 1) / gridDim.x);

  if (tid == 0) {
    for (int i = 0; i < kXStages; ++i) { mbar_init(smem_u32(&misc->full_x[i]), 1); mbar_init(smem_u32(&misc->empty_x[i]), 1); }
    for (int i = 0; i < kYStages; ++i) {
      mbar_init(smem_u32(&misc->d1_full[i]), 1);
      mbar_init(smem_u32(&misc->d1_empty[i]), nq1);  // one arrival per working warp of the Y-pass set on duty
      mbar_init(smem_u32(&misc->y_full[i]), nq1);
      mbar_init(smem_u32(&misc->y_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&misc->d2_full[i]), 1);
      mbar_init(smem_u32(&misc->d2_empty[i]), nh2 * nq2);  // one arrival per working warp of a quantize set
      mbar_init(smem_u32(&misc->set_sync[i]), nh2 * nq2);
    }
    for (int i = 0; i < 2 * 3 * 2 * 4; ++i) (&misc->absmax_part[0][0][0][0])[i] = 0.f;
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
    // core reads R as an N-major B operand (row k of R = one 128-byte row) and L as an M-major A operand (row k of L
    // laid along M, once per token copy), so nothing is transposed here.
    constexpr int kStagers = kThreads - 32;
    const int t13 = tid - 32;
    // Every thread first requests all its pieces of both transforms (one of R, at most two of LL) and only then stores
    // them: the loads come from L2 with several hundred cycles of latency each, and this staging is on the path of the
    // first group.
    // R: rows k < nc, 8 pieces per row; columns past nc are zero (the first product always has N = 64)
    // LL: rows k < k2 (rows m .. k2-1 pad the reduction length and must be zero), M position copy * mpad + i holds
    // L[k][i]; every other M position of these rows is zero.  M is a multiple of 8: pieces are whole or empty.
    static_assert(kStagers >= 64 * 8 && 2 * kStagers >= 64 * 16, "one piece of R and two of LL per thread cover the transforms");
    uint4 wr = make_uint4(0, 0, 0, 0), wl[2];
    {
      const int k = t13 >> 3, c = t13 & 7;
      if (t13 < nc * 8 && 8 * c < nc) wr = *reinterpret_cast<const uint4*>(right + k * nc + 8 * c);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int idx = t13 + j * kStagers, k = idx >> 4, c = idx & 15;
      const int cpy = (8 * c) / mpad, i0 = 8 * c - cpy * mpad;
      wl[j] = make_uint4(0, 0, 0, 0);
      if (idx < k2 * 16 && k < m && cpy < kGroup && i0 < m) wl[j] = *reinterpret_cast<const uint4*>(left + k * m + i0);
    }
    if (t13 < nc * 8) {
      const int k = t13 >> 3, c = t13 & 7;
      *reinterpret_cast<uint4*>(smem + kOffR + k * 128 + ((c ^ (k & 7)) << 4)) = wr;
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int idx = t13 + j * kStagers, k = idx >> 4, c = idx & 15;
      if (idx < k2 * 16) *reinterpret_cast<uint4*>(smem + kOffLL + (c >> 3) * (kAtomBytes / 2) + k * 128 + (((c & 7) ^ (k & 7)) << 4)) = wl[j];
    }
    if (k2 != m) {
      // M is not a multiple of 16: rows m .. k2-1 of each token's Y block only pad the reduction; they are zeroed once
      // (the Y pass never writes them)
      const int pad_rows = k2 - m, chunks = kYStages * kGroup * pad_rows * 8;
      for (int idx = t13; idx < chunks; idx += kStagers) {
        const int ch = idx & 7, pr = (idx >> 3) % pad_rows, blk = (idx >> 3) / pad_rows;  // blk = stage * kGroup + token
        const int row = (blk % kGroup) * k2 + m + pr;
        *reinterpret_cast<uint4*>(smem + kOffY + (blk / kGroup) * kStageBytes + row * 128 + (ch << 4)) = make_uint4(0, 0, 0, 0);
      }
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, %0;" ::"n"(kStagers) : "memory");
  }

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t bytes = (uint32_t)(rows_group * 128);
      int s = 0, ph = 0;
      long long grp = blockIdx.x;
      for (int it = 0; it < mine; ++it, grp += gridDim.x) {
        if (!mbar_wait(smem_u32(&misc->empty_x[s]), ph ^ 1)) { atomicCAS(status, 0u, 0x600u + s); break; }
        const uint32_t bar = smem_u32(&misc->full_x[s]);
        mbar_arrive_expect_tx(bar, bytes);
        tma_load_3d(smem_base + kOffX + s * kStageBytes, &x_map, bar, 0, 0, (int)(grp * kGroup));
        if (++s == kXStages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // One thread feeds the tensor core, so its instruction count per MMA matters: descriptors are built once and
      // advanced with a single add on the address field (units of 16 bytes).
      const uint32_t idesc1 = umma_idesc(1, Fmt<T>::id, Fmt<T>::id, 0, 1, 128, 64);  // B = R as it lies in memory: N-major
      const uint64_t desc_x0 = umma_smem_desc_sw128(smem_base + kOffX, 16, 1024);
      const uint64_t desc_r = umma_smem_desc_sw128(smem_base + kOffR, 16, 1024);      // one 64-column block; 16 rows of R = 2048 bytes per step
      int sx = 0, phx = 0, s1 = 0, ph1 = 0;
      for (int it = 0; it < mine; ++it) {
        if (const int w = mbar_wait2(smem_u32(&misc->full_x[sx]), phx, smem_u32(&misc->d1_empty[s1]), ph1 ^ 1)) {
          atomicCAS(status, 0u, 0x600u + 0x10u * w + sx);
          break;
        }
        tc_fence_after();
        const uint64_t da = desc_x0 + (uint64_t)(sx * (kStageBytes >> 4));
        if (FULL) {  // four back-to-back issues without loop overhead
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) mma_f16_ss(tmem + s1 * 64, da + ks * 2, desc_r + ks * 128, idesc1, ks);
        } else {
#pragma unroll 1
          for (int ks = 0; ks < (nc >> 4); ++ks) mma_f16_ss(tmem + s1 * 64, da + ks * 2, desc_r + ks * 128, idesc1, ks);
        }
        mma_commit(smem_u32(&misc->empty_x[sx]));
        mma_commit(smem_u32(&misc->d1_full[s1]));
        if (++sx == kXStages) { sx = 0; phx ^= 1; }
        if (++s1 == kYStages) { s1 = 0; ph1 ^= 1; }
      }
    }
  } else if (warp == 2) {
    // second-product issuer: its waits and commits overlap with the first-product MMAs of later groups
    if (lane == 0) {
      const uint32_t idesc2 = umma_idesc(1, Fmt<T>::id, Fmt<T>::id, 1, 1, 128, 128);  // A = LL, M-major
      const uint64_t desc_ll = umma_smem_desc_sw128(smem_base + kOffLL, kAtomBytes / 2, 1024);  // two 64-row blocks of 64 k-rows
      const uint64_t desc_y0 = umma_smem_desc_sw128(smem_base + kOffY, (uint32_t)(k2 * 128), 1024);  // N blocks = tokens, k2 rows apart
      const int ksteps2 = k2 >> 4;
      int sy = 0, phy = 0;
      for (int it = 0; it < mine; ++it) {
        const int e = it & 1, ph = (it >> 1) & 1;
        if (const int w = mbar_wait2(smem_u32(&misc->y_full[sy]), phy, smem_u32(&misc->d2_empty[e]), ph ^ 1)) {
          atomicCAS(status, 0u, 0x620u + 0x10u * w + sy);
          break;
        }
        tc_fence_after();
        uint64_t da2 = desc_ll, db2 = desc_y0 + (uint64_t)(sy * (kStageBytes >> 4));
#pragma unroll 1
        for (int ks = 0; ks < ksteps2; ++ks, da2 += 128, db2 += 128) mma_f16_ss(tmem + kColZ + e * 128, da2, db2, idesc2, ks);
        mma_commit(smem_u32(&misc->y_empty[sy]));
        mma_commit(smem_u32(&misc->d2_full[e]));
        if (++sy == kYStages) { sy = 0; phy ^= 1; }
      }
    }
  } else if (warp < kEpi2Warp0) {
    // ---- Y pass: set e (4 warps) takes the groups with (it & 1) == e; warp q converts lanes 32q .. 32q+31 ------------
    const int q = warp & 3, e = (warp - kEpi1Warp0) >> 2, r = q * 32 + lane;
    for (int it = e; it < (q < nq1 ? mine : 0); it += 2) {
      const int s = it % kYStages, ph = (it / kYStages) & 1;  // kYStages is even: a set sees every phase of its stages
      if (__any_sync(0xffffffffu, mbar_wait2(smem_u32(&misc->d1_full[s]), ph, smem_u32(&misc->y_empty[s]), ph ^ 1) != 0)) {
        atomicCAS(status, 0u, 0x700u + s);
        break;
      }
      tc_fence_after();
      const int yr = r < m ? r : r - m + k2;  // row of the Y stage: token c's rows start at c * k2
      // (rows start on 128-byte boundaries: piece c of the swizzled row is at (row | (yr & 7) << 4) ^ (c << 4), one logic
      // operation per store where (c ^ (yr & 7)) << 4 added to the row costs three; the Y pass shares the ALU pipe with the
      // quantize pass)
      const uint32_t yrow = (smem_base + kOffY + s * kStageBytes + yr * 128) | (uint32_t)((yr & 7) << 4);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + s * 64 + h * 32, v);
        tmem_ld_wait();
        if (h == 1) {
          tc_fence_before();
          mbar_arrive_warp(smem_u32(&misc->d1_empty[s]));  // accumulators are in registers: the stage can be overwritten
        }
        if (r < rows_group) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
            w.y = pack2<T>(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
            w.z = pack2<T>(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
            w.w = pack2<T>(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(yrow ^ (uint32_t)((h * 4 + j) << 4)), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
          }
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(smem_u32(&misc->y_full[s]));
    }
  } else {
    // ---- quantize pass ---------------------------------------------------------------------------------------
    // set e (8 warps) takes the groups with (it & 1) == e; warp (q, h) of a set works on columns 32h .. 32h+31 of lanes 32q ..
    const int e = (warp - kEpi2Warp0) >> 3, q = warp & 3, h = ((warp - kEpi2Warp0) >> 2) & 1, l = q * 32 + lane;
    const int c = l / mpad, mi = l - c * mpad;      // lane block c holds a copy of the Z rows: it serves token c
    const bool active = c < kGroup && mi < m;
    const int slot = ((q * 32 - c * mpad) >> 5) * 2 + h;  // this warp's index among the (at most 4) warps of its token
    const int feat = m * nc;
    const int cols = FULL ? 32 : min(32, max(0, nc - h * 32));  // real columns among this warp's 32 (a multiple of 16)
    long long grp = (long long)blockIdx.x + (long long)e * gridDim.x;
    const int mine_q = ((q * 32) / mpad < kGroup && q * 32 - ((q * 32) / mpad) * mpad < m && cols > 0) ? mine : 0;  // idle warps skip the pass
    for (int use = 0, it = e; it < mine_q; it += 2, ++use, grp += 2LL * gridDim.x) {
      const int ph = use & 1, buf = use % 3;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&misc->d2_full[e]), ph))) { atomicCAS(status, 0u, 0x800u + e); break; }
      tc_fence_after();
      const long long tok = grp * kGroup + c;
      const bool valid = active && tok < tokens;
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + kColZ + e * 128 + (active ? c : 0) * 64;
      uint32_t v[32];
      tmem_ld_32x32b_x32(taddr + h * 32, v);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(smem_u32(&misc->d2_empty[e]));  // the Z accumulators of this stage are free again

      // round Z to the activation dtype once, as packed pairs; both passes work on the pairs
      uint32_t zz[16];
      float s = 1.f, inv_s = 1.f;
      uint32_t rhi2 = 0, rlo2 = 0;  // 1/s as two packed terms of the activation dtype (bf16 only)
      bool clamp_needed = true;
      if (MODE != kTransform) {
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
        // every warp serves one token (copies start on warp boundaries): its maximum goes into the warp's own slot
        amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));  // non-negative floats order as integers
        if (lane == 0 && c < kGroup) misc->absmax_part[e][buf][c][slot] = amax;
        // the 128 threads of the set meet here (bounded); afterwards the slot holds the token's absmax
        const uint32_t gs = smem_u32(&misc->set_sync[e]);
        mbar_arrive_warp(gs);
        if (!__all_sync(0xffffffffu, mbar_wait(gs, ph))) { atomicCAS(status, 0u, 0x810u + e); break; }
        {
          // the slot buffer of this use is next written three uses later, after two more passes of this barrier
          const float4 p4 = *reinterpret_cast<const float4*>(&misc->absmax_part[e][buf][c < kGroup ? c : 0][0]);
          amax = fmaxf(fmaxf(p4.x, p4.y), fmaxf(p4.z, p4.w));
        }
        // max of the rounded values = rounded max; clip * absmax and the division by 7 are rounded like the reference.
        // top / 7 can neither hit nor come within 2^-13 (relative) of a midpoint of the 16-bit format, so the
        // float32 product with 1/7 rounds to the same 16-bit value as the exact quotient.
        const float top = rnd1<T>(amax * clip);  // amax already is a value of the activation dtype
        s = fmaxf(rnd1<T>(top * 0.142857149f), DT<T>::floor_scale());
        inv_s = __frcp_rn(s);
        P2<T>::recip2(inv_s, rhi2, rlo2);
        if (valid && mi == 0 && h == 0) store_scale(scales, tok, s, scale_dtype);
        // a quotient can only leave [-8, 7] after rounding if some |z| / s reaches 7.5; most warps have no such row
        clamp_needed = __any_sync(0xffffffffu, !(row_amax * inv_s < 7.4f));
      }
      const bool zero_scale = (MODE != kTransform) && (s == 0.f);

      {
        const int c0 = h * 32;
        if (MODE == kTransform) {
          if (valid) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + tok * feat + mi * nc + c0);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (4 * j < cols) dst[j] = make_float4(DT<T>::rnd(__uint_as_float(v[4 * j])), DT<T>::rnd(__uint_as_float(v[4 * j + 1])),
                                   DT<T>::rnd(__uint_as_float(v[4 * j + 2])), DT<T>::rnd(__uint_as_float(v[4 * j + 3])));
          }
        } else if (MODE == kPacked && !zero_scale) {
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
  auto kern = flatquant_n64_kernel<T, MODE, FULL>;
  int dev = 0, sms = 148;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    QO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[dev & 63] = true;
  }
  sms = sm_count(dev);
  const int64_t ngroups = (tokens + kGroup - 1) / kGroup;
  const int grid = (int)(ngroups < sms ? ngroups : sms);
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
                                 (long long)tokens, m, nc, clip, scale_dtype, status));
  return check_launch("flatquant_n64_kernel");
}

template <typename T>
int launch_mode(int mode, const CUtensorMap& map, const void* left, const void* right, void* out, void* scales,
                int64_t tokens, int m, int nc, float clip, int scale_dtype, uint32_t* status, cudaStream_t stream) {
  if (nc == 64) {
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

bool flatquant_sm100_n64_supported(int m, int n) { return n >= 16 && n <= 64 && (n % 16) == 0 && m >= 16 && m <= 64 && (m % 8) == 0; }

int launch_flatquant_sm100_n64(int mode, const void* x_map, const void* left, const void* right, void* out, void* scales,
                               int64_t tokens, int m, int n, float clip, int in_dtype, int scale_dtype, uint32_t* status,
                               cudaStream_t stream) {
  const CUtensorMap& map = *reinterpret_cast<const CUtensorMap*>(x_map);
  if (in_dtype == QO_BF16)
    return launch_mode<__nv_bfloat16>(mode, map, left, right, out, scales, tokens, m, n, clip, scale_dtype, status, stream);
  return launch_mode<__half>(mode, map, left, right, out, scales, tokens, m, n, clip, scale_dtype, status, stream);
}

}  // namespace qo
