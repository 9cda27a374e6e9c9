// FlatQuant quantizer for sm_100a: TMA in, both Kronecker products on tcgen05 tensor cores with the accumulators in
// tensor memory, scale + int4 codes straight from tensor memory to global memory with 16-byte stores.
//
// This is the shape-general kernel: it takes the N = 64 shapes whose M is not one of 16 / 32 / 48 / 64 (those run in
// flatquant_sm100_n64.cu; N = 128 runs in flatquant_sm100_n128.cu) and holds the host-side dispatch for all three.
//
// One persistent CTA per SM.  A tile is G = floor(128 / M) whole tokens, i.e. G*M <= 128 rows of N elements.
//
//   warp 0      TMA producer: 3-D tensor map (n, m, token) -> X tile rows in shared memory, 128-byte swizzle
//   warp 1      MMA issuer:   Y  = X . R          A = X tile (K-major),  B = R^T staged once (K-major)
//                             Z  = BD . Y         A = blockdiag(L^T) staged once (K-major), B = Y (N-major)
//   warps 2-5   Y pass:       tensor memory -> round to the activation dtype -> shared memory, as MMA operand
//   warps 6-13  two alternating groups of 4 warps: per-token absmax, scale, codes, stores
//
// blockdiag(L^T) puts the G copies of L^T on the diagonal of a 128 x 128 matrix, so one M=128 MMA transforms all
// tokens of the tile and the result keeps "one thread = one row of a token": the 8 nibbles of a packed word sit
// in one thread and rows of consecutive threads are contiguous in memory.
//
// The rounding points of the reference (src/quant_ops/ops/quantization/flatquant/ops.py:99-117) are kept: Y and Z
// are rounded to the activation dtype, so are clip*absmax, the division by 7 and the quotient z/scale.
// For clip > 0, max(|round(min*c)|, round(max*c)) equals round(c * max|z|) (rounding is odd and monotonic), so one
// running absmax is enough.  For bf16, round(z * (1/s)) equals round(z / s) exactly: z and s carry 8 significant
// bits, their quotient can neither hit nor come within 2^-17 (relative) of a midpoint between two bf16 values, and
// the float32 product is off by less than 2^-22.
//
// Every wait on an mbarrier is bounded; a wait that runs out stores a code in the status word and the CTA leaves.
#include <mutex>

#include "flatquant_sm100_common.cuh"

namespace qo {
namespace {

using namespace ptx;
using namespace fq;

constexpr int kThreads = 448;  // 14 warps


template <int NDIM>
struct Cfg {
  static constexpr int kAtoms = NDIM / 64;                // 64-element column blocks
  static constexpr int kXStages = NDIM == 64 ? 3 : 2;
  static constexpr int kXStageBytes = kAtoms * kAtomBytes;
  static constexpr int kYStageBytes = kAtoms * kAtomBytes;
  static constexpr int kRBytes = kAtoms * NDIM * 128;     // R^T, K-major: NDIM rows per K atom
  static constexpr int kBdBytes = 2 * kAtomBytes;         // blockdiag(L^T): 128 rows x up to 128 k
  static constexpr int kOffX = 0;
  static constexpr int kOffY = kOffX + kXStages * kXStageBytes;
  static constexpr int kOffR = kOffY + 2 * kYStageBytes;
  static constexpr int kOffBd = kOffR + kRBytes;
  static constexpr int kOffMisc = kOffBd + kBdBytes;
  static constexpr int kSmemBytes = kOffMisc + 1024 /*barriers, absmax slots*/ + 1024 /*alignment slack*/;
  static constexpr int kTmemCols = 512;                   // two stages each of Y and Z accumulators (+ blockdiag(L^T) for N = 64)
};

struct Misc {
  uint64_t full_x[3], empty_x[3];
  uint64_t d1_full[2], d1_empty[2], y_full[2], y_empty[2], d2_full[2], d2_empty[2];
  uint64_t group_sync[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  int absmax_bits[2][3][8];
};


__device__ __forceinline__ void report(uint32_t* status, Misc* misc, uint32_t code) {
  atomicCAS(status, 0u, code);
  atomicExch(&misc->abort_flag, 1u);
}

template <typename T, int NDIM, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
flatquant_sm100_kernel(const __grid_constant__ CUtensorMap x_map, const T* __restrict__ left,
                       const T* __restrict__ right, void* __restrict__ out, void* __restrict__ scales,
                       long long tokens, int m, float clip, int scale_dtype, uint32_t* __restrict__ status) {
  using C = Cfg<NDIM>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + C::kOffMisc);
  const uint32_t smem_base = smem_u32(smem);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g_tokens = 128 / m;           // tokens per tile
  const int rows_tile = g_tokens * m;     // valid rows per tile
  const int k2 = (rows_tile + 15) & ~15;  // reduction length of the second product
  const long long ntiles = (tokens + g_tokens - 1) / g_tokens;

  // ---- one-time set-up ---------------------------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) { mbar_init(smem_u32(&misc->full_x[i]), 1); mbar_init(smem_u32(&misc->empty_x[i]), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&misc->d1_full[i]), 1);
      mbar_init(smem_u32(&misc->d1_empty[i]), 128);
      mbar_init(smem_u32(&misc->y_full[i]), 128);
      mbar_init(smem_u32(&misc->y_empty[i]), 1);
      mbar_init(smem_u32(&misc->d2_full[i]), 1);
      mbar_init(smem_u32(&misc->d2_empty[i]), 128);
      mbar_init(smem_u32(&misc->group_sync[i]), 128);
    }
    misc->abort_flag = 0;
    for (int i = 0; i < 2 * 3 * 8; ++i) (&misc->absmax_bits[0][0][0])[i] = 0;
    fence_barrier_init();
    prefetch_tensormap(&x_map);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&misc->tmem_base), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();  // barriers and the tensor-memory base exist; the producer can start filling the X stages
  tc_fence_after();
  const uint32_t tmem = misc->tmem_base;

  // blockdiag(L^T) lives in tensor memory when there is room beside the accumulators (N = 64), else in shared memory
  constexpr bool kBdInTmem = (NDIM == 64);
  const uint32_t tmem_bd = tmem + 4 * NDIM;

  if (warp != 0) {
    constexpr int kStagers = kThreads - 32;  // warps 1-13
    const int t13 = tid - 32;
    // Step 1: raw copies of L and R into shared memory that nothing uses yet, 16-byte loads all in flight at once.
    T* raw_l = reinterpret_cast<T*>(smem + (kBdInTmem ? C::kOffBd : C::kOffY));
    T* raw_r = reinterpret_cast<T*>(smem + (kBdInTmem ? C::kOffY : C::kOffY + C::kYStageBytes));
    {
      const int l_chunks = (m * m) / 8, r_chunks = NDIM * NDIM / 8;
      constexpr int kMaxIter = (2 * 128 * 128 / 8 + kStagers - 1) / kStagers;
      uint4 tmp[kMaxIter];
#pragma unroll
      for (int i = 0; i < kMaxIter; ++i) {
        const int c = t13 + i * kStagers;
        if (c < l_chunks) tmp[i] = reinterpret_cast<const uint4*>(left)[c];
        else if (c - l_chunks < r_chunks) tmp[i] = reinterpret_cast<const uint4*>(right)[c - l_chunks];
      }
#pragma unroll
      for (int i = 0; i < kMaxIter; ++i) {
        const int c = t13 + i * kStagers;
        if (c < l_chunks) reinterpret_cast<uint4*>(raw_l)[c] = tmp[i];
        else if (c - l_chunks < r_chunks) reinterpret_cast<uint4*>(raw_r)[c - l_chunks] = tmp[i];
      }
      for (int i = l_chunks * 8 + t13; i < m * m; i += kStagers) raw_l[i] = left[i];  // tail when m*m is not a multiple of 8
      if (!kBdInTmem)
        for (int idx = t13; idx < C::kBdBytes / 16; idx += kStagers) reinterpret_cast<uint4*>(smem + C::kOffBd)[idx] = make_uint4(0, 0, 0, 0);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kStagers) : "memory");

    // Step 2: operands in the layouts the MMAs read.
    if (kBdInTmem && warp >= 2 && warp < 6) {
      // lane r of tensor memory = row r of blockdiag(L^T); 32-bit column j holds k = 2j (low half) and 2j + 1
      const int q = warp & 3, r = q * 32 + lane;
      const int gg = r / m, i = r - gg * m, c_lo = gg * m;
      const bool row_ok = r < rows_tile;
      const uint16_t* rl = reinterpret_cast<const uint16_t*>(raw_l);
#pragma unroll
      for (int cb = 0; cb < 64; cb += 8) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int k0 = 2 * (cb + j) - c_lo, k1 = k0 + 1;
          const uint32_t v0 = (row_ok && k0 >= 0 && k0 < m) ? rl[k0 * m + i] : 0u;
          const uint32_t v1 = (row_ok && k1 >= 0 && k1 < m) ? rl[k1 * m + i] : 0u;
          w[j] = v0 | (v1 << 16);
        }
        tmem_st_32x32b_x8(tmem_bd + ((uint32_t)(q * 32) << 16) + cb, w);
      }
      tmem_st_wait();
    } else {
      // R^T as a K-major operand: row = output column n, k = j runs along the row, 128-byte swizzle per 8 rows
      const int first = kBdInTmem ? (warp == 1 ? lane : (warp - 5) * 32 + lane) : t13;  // dense index over the warps here
      constexpr int kWorkers = kBdInTmem ? kStagers - 128 : kStagers;
      for (int c = first; c < NDIM * NDIM / 8; c += kWorkers) {
        const int j = c / (NDIM / 8), n0 = (c % (NDIM / 8)) * 8;  // R[j][n0 .. n0+7]
        const uint4 v = reinterpret_cast<const uint4*>(raw_r)[c];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e8 = 0; e8 < 8; ++e8) {
          const int n = n0 + e8;
          const uint32_t off = (j >> 6) * (NDIM * 128) + (n >> 3) * 1024 + (n & 7) * 128 + ((((j & 63) >> 3) ^ (n & 7)) << 4) + (j & 7) * 2;
          *reinterpret_cast<uint16_t*>(smem + C::kOffR + off) = (uint16_t)(w[e8 >> 1] >> (16 * (e8 & 1)));
        }
      }
      if (!kBdInTmem) {
        // diagonal blocks of blockdiag(L^T) in shared memory: entry (row (g, i), column (g, k)) = L[k][i]
        const uint16_t* rl = reinterpret_cast<const uint16_t*>(raw_l);
        for (int idx = t13; idx < rows_tile * m; idx += kStagers) {
          const int gk = idx / m, i = idx - gk * m;  // gk = g * m + k = the column
          const int gg = gk / m, r = gg * m + i, c = gk;
          const uint32_t off = (c >> 6) * kAtomBytes + (r >> 3) * 1024 + (r & 7) * 128 + ((((c & 63) >> 3) ^ (r & 7)) << 4) + (c & 7) * 2;
          *reinterpret_cast<uint16_t*>(smem + C::kOffBd + off) = rl[(gk - gg * m) * m + i];
        }
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(kStagers) : "memory");
    tc_fence_after();
  }

  // ---- roles ---------------------------------------------------------------------------------------
  if (warp == 0) {
    if (lane == 0) {
      const uint32_t tile_bytes = (uint32_t)(C::kAtoms * 64 * m * g_tokens * sizeof(T));
      int it = 0;
      for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
        const int s = it % C::kXStages, ph = (it / C::kXStages) & 1;
        if (!mbar_wait(smem_u32(&misc->empty_x[s]), ph ^ 1)) { report(status, misc, 0x100 + s); break; }
        const uint32_t bar = smem_u32(&misc->full_x[s]);
        mbar_arrive_expect_tx(bar, tile_bytes);
#pragma unroll
        for (int a = 0; a < C::kAtoms; ++a)
          tma_load_3d(smem_base + C::kOffX + s * C::kXStageBytes + a * kAtomBytes, &x_map, bar, 64 * a, 0,
                      (int)(tile * g_tokens));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc1 = umma_idesc(1, Fmt<T>::id, Fmt<T>::id, 0, 0, 128, NDIM);
      const uint32_t idesc2 = umma_idesc(1, Fmt<T>::id, Fmt<T>::id, 0, 1, 128, NDIM);
      // Y as an N-major B operand: 64-column blocks one atom apart (leading offset), 8-row k groups 1024 bytes apart
      constexpr uint32_t y_lbo = (uint32_t)kAtomBytes, y_sbo = 1024u;
      long long my_tiles = 0;
      if ((long long)blockIdx.x < ntiles) my_tiles = (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
      bool ok = true;
      auto first_product = [&](long long it) -> bool {
        const int sx = (int)(it % C::kXStages), phx = (int)((it / C::kXStages) & 1);
        const int s1 = (int)(it & 1), ph1 = (int)((it >> 1) & 1);
        if (!mbar_wait(smem_u32(&misc->full_x[sx]), phx)) { report(status, misc, 0x200 + sx); return false; }
        if (!mbar_wait(smem_u32(&misc->d1_empty[s1]), ph1 ^ 1)) { report(status, misc, 0x210 + s1); return false; }
        tc_fence_after();
        const uint32_t a_base = smem_base + C::kOffX + sx * C::kXStageBytes, b_base = smem_base + C::kOffR;
#pragma unroll
        for (int ks = 0; ks < NDIM / 16; ++ks) {
          const uint64_t ad = umma_smem_desc_sw128(a_base + (ks >> 2) * kAtomBytes + (ks & 3) * 32, 16, 1024);
          const uint64_t bd = umma_smem_desc_sw128(b_base + (ks >> 2) * (NDIM * 128) + (ks & 3) * 32, 16, 1024);
          mma_f16_ss(tmem + s1 * NDIM, ad, bd, idesc1, ks > 0);
        }
        mma_commit(smem_u32(&misc->empty_x[sx]));
        mma_commit(smem_u32(&misc->d1_full[s1]));
        return true;
      };
      auto second_product = [&](long long it) -> bool {
        const int s = (int)(it & 1), ph = (int)((it >> 1) & 1);
        if (!mbar_wait(smem_u32(&misc->y_full[s]), ph)) { report(status, misc, 0x220 + s); return false; }
        if (!mbar_wait(smem_u32(&misc->d2_empty[s]), ph ^ 1)) { report(status, misc, 0x230 + s); return false; }
        tc_fence_after();
        const uint32_t a_base = smem_base + C::kOffBd, b_base = smem_base + C::kOffY + s * C::kYStageBytes;
        for (int ks = 0; ks < k2 / 16; ++ks) {
          const uint64_t bd = umma_smem_desc_sw128(b_base + ks * 2048, y_lbo, y_sbo);
          if (kBdInTmem) {
            mma_f16_ts(tmem + (2 + s) * NDIM, tmem_bd + ks * 8, bd, idesc2, ks > 0);  // 16 k = 8 packed columns
          } else {
            const uint64_t ad = umma_smem_desc_sw128(a_base + (ks >> 2) * kAtomBytes + (ks & 3) * 32, 16, 1024);
            mma_f16_ss(tmem + (2 + s) * NDIM, ad, bd, idesc2, ks > 0);
          }
        }
        mma_commit(smem_u32(&misc->y_empty[s]));
        mma_commit(smem_u32(&misc->d2_full[s]));
        return true;
      };
      if (my_tiles > 0) ok = first_product(0);
      for (long long it = 0; ok && it < my_tiles; ++it) {
        if (it + 1 < my_tiles) ok = first_product(it + 1);
        if (ok) ok = second_product(it);
      }
    }
  } else if (warp < 6) {
    // ---- Y pass: row r of the tile = tensor-memory lane r ----------------------------------------
    const int q = warp & 3, r = q * 32 + lane;
    int it = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int s = it & 1, ph = (it >> 1) & 1;
      // (outcomes are made warp-uniform: the tensor-memory loads below are warp-collective)
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&misc->d1_full[s]), ph))) { report(status, misc, 0x300 + s); break; }
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&misc->y_empty[s]), ph ^ 1))) { report(status, misc, 0x310 + s); break; }
      tc_fence_after();
      uint8_t* yrow = smem + C::kOffY + s * C::kYStageBytes + r * 128;
#pragma unroll
      for (int c0 = 0; c0 < NDIM; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + s * NDIM + c0, v);
        tmem_ld_wait();
        if (r < k2) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            if (r < rows_tile) {
              w.x = pack2<T>(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
              w.y = pack2<T>(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              w.z = pack2<T>(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              w.w = pack2<T>(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            } else {
              w = make_uint4(0, 0, 0, 0);  // rows that only pad the reduction length must be exact zeros
            }
            const int chunk = (c0 >> 3) + j;  // 16-byte chunk along N
            *reinterpret_cast<uint4*>(yrow + (chunk >> 3) * kAtomBytes + (((chunk & 7) ^ (r & 7)) << 4)) = w;
          }
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&misc->d1_empty[s]));
      mbar_arrive(smem_u32(&misc->y_full[s]));
    }
  } else {
    // ---- quantize pass: group e takes the tiles with (it & 1) == e --------------------------------
    const int e = (warp - 6) >> 2, q = warp & 3, r = q * 32 + lane;
    const int g = r / m, mi = r - g * m;
    const bool warp_uniform = (g_tokens == 1) || ((m & 31) == 0);
    const int feat = m * NDIM;
    constexpr bool kHold = (NDIM == 64) && (MODE != kTransform);  // whole row stays in registers between the passes
    int it = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      if ((it & 1) != e) continue;
      const int use = it >> 1, ph = use & 1, buf = use % 3;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&misc->d2_full[e]), ph))) { report(status, misc, 0x400 + e); break; }
      tc_fence_after();
      const long long tok = tile * g_tokens + g;
      const bool valid = r < rows_tile && tok < tokens;
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (2 + e) * NDIM;

      uint32_t held[kHold ? 2 : 1][32];
      float amax = 0.f;
      if (MODE != kTransform) {
        if (kHold) {
          tmem_ld_32x32b_x32(taddr, held[0]);
          tmem_ld_32x32b_x32(taddr + 32, held[kHold ? 1 : 0]);
          tmem_ld_wait();
          tc_fence_before();
          mbar_arrive(smem_u32(&misc->d2_empty[e]));  // accumulator stage is free again
#pragma unroll
          for (int i = 0; i < 32; ++i)
            amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(held[0][i])), fabsf(__uint_as_float(held[kHold ? 1 : 0][i]))));
        } else {
#pragma unroll
          for (int c0 = 0; c0 < NDIM; c0 += 32) {
            tmem_ld_32x32b_x32(taddr + c0, held[0]);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(__uint_as_float(held[0][i])));
          }
        }
        if (!valid) amax = 0.f;
        amax = DT<T>::rnd(amax);  // max of the rounded values = rounded max
        if (warp_uniform) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          if (lane == 0 && r < rows_tile) atomicMax(&misc->absmax_bits[e][buf][g], __float_as_int(amax));
        } else if (r < rows_tile) {
          atomicMax(&misc->absmax_bits[e][buf][g], __float_as_int(amax));
        }
        // all 128 threads of the group meet here (bounded), then the slot holds the token's absmax
        const uint32_t gs = smem_u32(&misc->group_sync[e]);
        mbar_arrive(gs);
        if (!__all_sync(0xffffffffu, mbar_wait(gs, ph))) { report(status, misc, 0x410 + e); break; }
        if (r < rows_tile) amax = __int_as_float(misc->absmax_bits[e][buf][g]);
        if (tid - (6 + 4 * e) * 32 < 8) misc->absmax_bits[e][(use + 2) % 3][tid - (6 + 4 * e) * 32] = 0;
      }

      float s = 1.f, inv_s = 1.f;
      if (MODE != kTransform) {
        const float top = DT<T>::rnd(amax * clip);
        s = fmaxf(DT<T>::rnd(__fdiv_rn(top, 7.0f)), DT<T>::floor_scale());
        inv_s = __frcp_rn(s);
        if (valid && mi == 0) store_scale(scales, tok, s, scale_dtype);
      }
      const bool zero_scale = (MODE != kTransform) && (s == 0.f);  // fp16 only: all-zero (or all-subnormal) row

#pragma unroll
      for (int c0 = 0; c0 < NDIM; c0 += 32) {
        uint32_t(&v)[32] = held[kHold ? (c0 >> 5) : 0];
        if (!kHold) {
          tmem_ld_32x32b_x32(taddr + c0, v);
          tmem_ld_wait();
        }
        if (MODE == kTransform) {
          if (valid) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + tok * feat + mi * NDIM + c0);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              dst[j] = make_float4(DT<T>::rnd(__uint_as_float(v[4 * j])), DT<T>::rnd(__uint_as_float(v[4 * j + 1])),
                                   DT<T>::rnd(__uint_as_float(v[4 * j + 2])), DT<T>::rnd(__uint_as_float(v[4 * j + 3])));
          }
        } else {
          uint32_t pb[4], qb[4];  // nibble-bytes of the 32 elements, 4 + 4 per group of 8
          if (!zero_scale) {
#pragma unroll
            for (int j = 0; j < 4; ++j) nibble_bytes<T>(v, 8 * j, s, inv_s, pb[j], qb[j]);
          } else {
            // the reference divides by zero here: +-inf clamps to 7 / -8, 0/0 counts as 0
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              pb[j] = qb[j] = 0;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float z0 = DT<T>::rnd(__uint_as_float(v[8 * j + i])), z1 = DT<T>::rnd(__uint_as_float(v[8 * j + 4 + i]));
                pb[j] |= (uint32_t)(z0 > 0.f ? 15 : (z0 < 0.f ? 0 : 8)) << (8 * i);
                qb[j] |= (uint32_t)(z1 > 0.f ? 15 : (z1 < 0.f ? 0 : 8)) << (8 * i);
              }
            }
          }
          if (MODE == kPacked) {
            if (valid) {
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(out) + tok * (feat / 8) + (mi * NDIM + c0) / 8);
              *dst = make_uint4(pack8(pb[0], qb[0]), pack8(pb[1], qb[1]), pack8(pb[2], qb[2]), pack8(pb[3], qb[3]));
            }
          } else if (valid) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<int8_t*>(out) + tok * feat + mi * NDIM + c0);
            dst[0] = make_uint4(bytes4(pb[0]), bytes4(qb[0]), bytes4(pb[1]), bytes4(qb[1]));
            dst[1] = make_uint4(bytes4(pb[2]), bytes4(qb[2]), bytes4(pb[3]), bytes4(qb[3]));
          }
        }
      }
      if (!kHold) {
        tc_fence_before();
        mbar_arrive(smem_u32(&misc->d2_empty[e]));
      }
    }
  }

  // ---- teardown ----------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// ---- host side ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

std::mutex g_status_mu;
uint32_t* g_status_words[64] = {};

uint32_t* status_word(int dev) {
  std::mutex& mu = g_status_mu;
  uint32_t** words = g_status_words;
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!words[dev]) {
    if (cudaMalloc(&words[dev], sizeof(uint32_t)) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    cudaMemset(words[dev], 0, sizeof(uint32_t));
  }
  return words[dev];
}

template <typename T, int NDIM, int MODE>
int launch_one(const CUtensorMap& map, const void* left, const void* right, void* out, void* scales, int64_t tokens,
               int m, float clip, int scale_dtype, uint32_t* status, cudaStream_t stream) {
  using C = Cfg<NDIM>;
  auto kern = flatquant_sm100_kernel<T, NDIM, MODE>;
  int dev = 0, sms = 148;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  static bool configured[64] = {};  // per instantiation and device
  if (!configured[dev & 63]) {
    QO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured[dev & 63] = true;
  }
  sms = sm_count(dev);
  const int g = 128 / m;
  const int64_t ntiles = (tokens + g - 1) / g;
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(map, reinterpret_cast<const T*>(left), reinterpret_cast<const T*>(right),
                                                  out, scales, (long long)tokens, m, clip, scale_dtype, status);
  return check_launch("flatquant_sm100_kernel");
}

template <typename T, int NDIM>
int launch_mode(int mode, const CUtensorMap& map, const void* left, const void* right, void* out, void* scales,
                int64_t tokens, int m, float clip, int scale_dtype, uint32_t* status, cudaStream_t stream) {
  switch (mode) {
    case kInt8: return launch_one<T, NDIM, kInt8>(map, left, right, out, scales, tokens, m, clip, scale_dtype, status, stream);
    case kPacked: return launch_one<T, NDIM, kPacked>(map, left, right, out, scales, tokens, m, clip, scale_dtype, status, stream);
    default: return launch_one<T, NDIM, kTransform>(map, left, right, out, scales, tokens, m, clip, scale_dtype, status, stream);
  }
}

}  // namespace

uint32_t* device_status_word(int dev) { return status_word(dev); }
uint32_t* device_status_word_if_any(int dev) {
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mu);
  return g_status_words[dev];
}

bool flatquant_sm100_supported(int64_t ldx, int m, int n, int in_dtype, const void* x, const void* left, const void* right,
                               float clip) {
  if (in_dtype != QO_F16 && in_dtype != QO_BF16) return false;
  if (!(clip > 0.f)) return false;                            // the single running absmax needs a positive clip ratio
  if (n != 64 && !flatquant_sm100_n128_supported(m, n) && !flatquant_sm100_n64_supported(m, n)) return false;
  if (m < 16 || m > 128) return false;
  if (ldx % 8) return false;                                  // TMA: row stride must be a multiple of 16 bytes
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(left) % 16 || reinterpret_cast<uintptr_t>(right) % 16) return false;
  return encode_fn() != nullptr;
}

// mode: 0 int8 codes, 1 packed codes, 2 transform only (float32 Z written to `codes`)
int launch_flatquant_sm100_mode(int mode, const void* x, int64_t ldx, const void* left, const void* right, void* codes,
                                void* scales, int64_t tokens, int m, int n, float clip, int in_dtype, int scale_dtype,
                                cudaStream_t stream) {
  if (reinterpret_cast<uintptr_t>(codes) % 16) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: output pointer must be 16-byte aligned");
  if (tokens * (int64_t)1 > 0x7fffffffLL) return fail(QO_ERR_UNSUPPORTED, "flatquant: more than 2^31 tokens in one call");
  int dev = 0;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  uint32_t* status = status_word(dev);
  if (!status) return fail(QO_ERR_CUDA, "flatquant: could not allocate the device status word");

  CUtensorMap map;
  const cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)tokens};
  const cuuint64_t strides[2] = {(cuuint64_t)n * 2, (cuuint64_t)ldx * 2};
  const bool batched = flatquant_sm100_n64_supported(m, n);  // groups of 2 tokens, stacked-L^T second product
  const bool wide = flatquant_sm100_n128_supported(m, n);     // right transform of size 128
  const cuuint32_t box[3] = {64, (cuuint32_t)m, (cuuint32_t)(batched ? 2 : (wide ? flatquant_sm100_n128_group(m) : 128 / m))};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode_fn()(&map, in_dtype == QO_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                 3, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QO_ERR_CUDA, "flatquant: cuTensorMapEncodeTiled failed with code %d", (int)r);

  if (batched)
    return launch_flatquant_sm100_n64(mode, &map, left, right, codes, scales, tokens, m, n, clip, in_dtype, scale_dtype, status, stream);
  if (wide)
    return launch_flatquant_sm100_n128(mode, &map, left, right, codes, scales, tokens, m, n, clip, in_dtype, scale_dtype, status, stream);
  if (in_dtype == QO_BF16)
    return launch_mode<__nv_bfloat16, 64>(mode, map, left, right, codes, scales, tokens, m, clip, scale_dtype, status, stream);
  return launch_mode<__half, 64>(mode, map, left, right, codes, scales, tokens, m, clip, scale_dtype, status, stream);
}

int launch_flatquant_sm100(const void* x, int64_t ldx, const void* left, const void* right, void* codes, void* scales,
                           int64_t tokens, int m, int n, float clip, int in_dtype, int pack, int scale_dtype,
                           cudaStream_t stream) {
  return launch_flatquant_sm100_mode(pack ? kPacked : kInt8, x, ldx, left, right, codes, scales, tokens, m, n, clip,
                                     in_dtype, scale_dtype, stream);
}

}  // namespace qo
