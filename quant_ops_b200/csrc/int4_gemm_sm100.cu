// Packed-int4 GEMM for sm_100a.
//
// Two steps on the caller's stream:
//   1. widen: each packed operand is rewritten once as signed bytes into the workspace: A8 [T, K] row-major, B8 in
//      blocks of 256 output channels x 128 K-bytes (32 KB each, ordered [Nout / 256][K / 128]), so that every B
//      slice the GEMM fetches is one contiguous piece of memory instead of 256 pieces of 128 bytes, K bytes apart
//      (short activation matrices stream the weights from HBM exactly once).  Doing this in a pass of its own keeps
//      the GEMM main loop free of ALU work and of extra shared-memory traffic; the bytes written stay in the 126 MB
//      L2 for the GEMM that follows.
//   2. GEMM: persistent CTAs, one 128 x BN output tile at a time.  Warp 0 streams 128-byte-wide K slices of A8 and
//      B8 with TMA (128-byte swizzle) through a ring of shared-memory stages, warp 1 issues tcgen05.mma kind::i8
//      (int8 x int8 -> int32) into tensor memory, warps 2-5 read the accumulators back, apply
//      (float(acc) * scale_a[row]) * scale_b[col] and store fp16 / bf16.  Two accumulator stages in tensor memory
//      let the epilogue of one tile overlap the main loop of the next.  Short activation matrices split K over the
//      2, 4 or 8 CTAs of a thread-block cluster, which add their partial sums through distributed shared memory.
//
// Arithmetic is that of the reference kernel (src/quant_ops/ops/quantization/int4_matmul/kernels/
// cuda_int4_matmul_kernel.cu:104-116): exact int32 accumulation, then the two float32 multiplies in that order.
// Every mbarrier wait is bounded; a wait that runs out records a code in the device status word.  The cluster barriers
// of the K-split are hardware barriers that every thread reaches on every path (no thread returns early).
#include <mutex>
#include <type_traits>

#include "qo_internal.cuh"
#include "sm100_ptx.cuh"

namespace qo {
namespace {

using namespace ptx;

constexpr int kBM = 128;       // rows per output tile
constexpr int kBK = 128;       // K bytes per pipeline stage (one 128-byte swizzle atom)
constexpr int kGemmThreads = 192;

// ---- step 1: widen ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint2 widen8(uint32_t w) {
  const uint32_t even = w & 0x0F0F0F0Fu, odd = (w >> 4) & 0x0F0F0F0Fu;
  const uint32_t l = __byte_perm(even, odd, 0x5140), h = __byte_perm(even, odd, 0x7362);
  return make_uint2(((l | 0x80808080u) - 0x08080808u) ^ 0x80808080u, ((h | 0x80808080u) - 0x08080808u) ^ 0x80808080u);
}

// Byte offset of element (row, kbyte) of a widened operand.  ksteps == 0: row-major with row length k (the A operand);
// otherwise the blocked layout of the B operand, ksteps = ceil(K / 128) blocks per 256 rows.
__device__ __forceinline__ int64_t widened_offset(int64_t row, int64_t kbyte, int64_t k, int64_t ksteps) {
  if (ksteps == 0) return row * k + kbyte;
  return (((row >> 8) * ksteps + (kbyte >> 7)) << 15) + ((row & 255) << 7) + (kbyte & 127);
}

// rows of packed words with unit stride along K, 8 bytes out per thread
__global__ void __launch_bounds__(256)
widen_rows_kernel(const uint32_t* __restrict__ in, int64_t ld_words, uint8_t* __restrict__ out, int64_t rows, int64_t kwords,
                  int64_t ksteps) {
  const int64_t total = rows * kwords;
  for (int64_t i = blockIdx.x * 256LL + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t r = i / kwords, kw = i - r * kwords;
    *reinterpret_cast<uint2*>(out + widened_offset(r, 8 * kw, 8 * kwords, ksteps)) = widen8(in[r * ld_words + kw]);
  }
}

// The same for up to two operands in one launch, 16 bytes in and 32 bytes out per thread (rows 16-byte aligned,
// K a multiple of 32): both operands of a GEMM are widened by one kernel.
struct WidenJob {
  const uint32_t* in;
  uint8_t* out;
  int64_t ld_words, rows, kquads;  // kquads = K / 32 = groups of four packed words per row
  int64_t ksteps;                  // 0: row-major output, else the blocked layout
};
// chained: the kernel was launched with programmatic stream serialization behind a kernel whose output it does not
// touch (the fused layer: the activation quantizer, while this pass widens the weights), so it runs beside that
// kernel; before it ends it waits for that kernel, so that whoever waits for this one has waited for both.
__global__ void __launch_bounds__(256)
widen_rows2_kernel(WidenJob j0, WidenJob j1, int chained) {
  grid_launch_dependents();  // the GEMM that follows may set itself up; it waits before it reads anything
  const int64_t n0 = j0.rows * j0.kquads, total = n0 + j1.rows * j1.kquads;
  for (int64_t i = blockIdx.x * 256LL + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const bool second = i >= n0;
    const WidenJob& j = second ? j1 : j0;
    const int64_t e = second ? i - n0 : i;
    const int64_t r = e / j.kquads, q = e - r * j.kquads;
    const uint4 w = *reinterpret_cast<const uint4*>(j.in + r * j.ld_words + q * 4);
    const uint2 a = widen8(w.x), b = widen8(w.y), c = widen8(w.z), d = widen8(w.w);
    uint4* o = reinterpret_cast<uint4*>(j.out + widened_offset(r, 32 * q, 32 * j.kquads, j.ksteps));
    o[0] = make_uint4(a.x, a.y, b.x, b.y);
    o[1] = make_uint4(c.x, c.y, d.x, d.y);
  }
  if (chained) grid_dependency_wait();
}

// reference B layout [K/8, N] with N contiguous: transpose 32 x 32 words through shared memory so that the reads run
// along N and the writes along K; the output is the blocked layout
__global__ void __launch_bounds__(256)
widen_transpose_kernel(const uint32_t* __restrict__ in, int64_t bsk, int64_t bsn, uint8_t* __restrict__ out, int64_t n,
                       int64_t kwords, int64_t ksteps) {
  __shared__ uint2 tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t n0 = (int64_t)blockIdx.x * 32, k0 = (int64_t)blockIdx.y * 32;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t kw = k0 + ty + 8 * i, col = n0 + tx;
    uint32_t w = 0x88888888u;
    if (kw < kwords && col < n) w = in[kw * bsk + col * bsn];
    tile[ty + 8 * i][tx] = widen8(w);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t col = n0 + ty + 8 * i, kw = k0 + tx;
    if (col < n && kw < kwords) *reinterpret_cast<uint2*>(out + widened_offset(col, 8 * kw, 8 * kwords, ksteps)) = tile[tx][ty + 8 * i];
  }
}

// ---- step 2: GEMM --------------------------------------------------------------------------------------------
// The blocked B operand seen as a matrix of 128-byte rows: first row of the slice (channels n0 .., K step ks)
__device__ __forceinline__ int b_block_row(int n0, int ks, int ksteps) { return ((n0 >> 8) * ksteps + ks) * 256 + (n0 & 255); }

template <int BN>
struct GemmCfg {
  static constexpr int kStageBytes = (kBM + BN) * kBK;
  static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kOffSb = kStages * kStageBytes;           // 4 warps x BN floats
  static constexpr int kOffBar = kOffSb + 4 * BN * 4;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
};

struct GemmBars {
  uint64_t full[8], empty[8], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};

template <typename OutT>
__device__ __forceinline__ uint32_t pack_out2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_out2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_out2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_out2(uint32_t w, __half) {
  return __half22float2(*reinterpret_cast<__half2*>(&w));
}
__device__ __forceinline__ float2 unpack_out2(uint32_t w, __nv_bfloat16) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_s8_sm100_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                     const float* __restrict__ sa, const float* __restrict__ sb, OutT* __restrict__ out,
                     int32_t* __restrict__ acc_out, const OutT* __restrict__ bias, int t, int n, int k, int ksplit,
                     int b_early, uint32_t* __restrict__ status) {
  using C = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmBars* bars = reinterpret_cast<GemmBars*>(smem + C::kOffBar);
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_n = (n + BN - 1) / BN, tiles_m = (t + kBM - 1) / kBM;
  // A work item is an output tile and one of `ksplit` slices of K.  With ksplit > 1 the kernel is launched as
  // clusters of ksplit CTAs with one work item each (cluster rank = K slice): every CTA of the cluster collects the
  // slices' int32 partial sums of 128 / ksplit rows of the tile in its shared memory, sums them and writes the outputs.
  const int ntiles = tiles_m * tiles_n * ksplit, ksteps = (k + kBK - 1) / kBK;

  if (tid == 0) {
    for (int i = 0; i < C::kStages; ++i) { mbar_init(smem_u32(&bars->full[i]), 1); mbar_init(smem_u32(&bars->empty[i]), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&bars->acc_full[i]), 1); mbar_init(smem_u32(&bars->acc_empty[i]), 128); }
    fence_barrier_init();
    prefetch_tensormap(&a_map);
    prefetch_tensormap(&b_map);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  // Launched with programmatic stream serialization: the set-up above may overlap the tail of the preceding kernel
  // of the stream (the quantizer or the widening pass); nothing below reads or writes global memory before it is done.
  // One exception, b_early: the caller says that B was not written by that kernel (weights prepared at load time,
  // the predecessor is this call's quantizer, which releases its dependents only after its own dependency wait), so
  // the B halves of the first stages are requested before the wait and their HBM latency overlaps it.
  int early = 0;  // stages of the first work item whose B half is already on its way
  if (b_early && warp == 0 && lane == 0 && blockIdx.x < ntiles) {
    const int item = blockIdx.x, tile = item / ksplit, kz = item - tile * ksplit;
    const int nb = tile % tiles_n;
    const int ks0 = (int)((long long)kz * ksteps / ksplit), ks1 = (int)((long long)(kz + 1) * ksteps / ksplit);
    early = min(C::kStages, ks1 - ks0);
    for (int s = 0; s < early; ++s) {
      const uint32_t bar = smem_u32(&bars->full[s]);
      mbar_arrive_expect_tx(bar, C::kStageBytes);
      tma_load_2d(smem_base + s * C::kStageBytes + kBM * kBK, &b_map, bar, 0, b_block_row(nb * BN, ks0 + s, ksteps));
    }
  }
  grid_dependency_wait();

  if (warp == 0) {
    if (lane == 0) {
      int step = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < ntiles; item += gridDim.x) {
        const int tile = item / ksplit, kz = item - tile * ksplit;
        const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
        const int ks0 = (int)((long long)kz * ksteps / ksplit), ks1 = (int)((long long)(kz + 1) * ksteps / ksplit);
        for (int ks = ks0; ks < ks1; ++ks, ++step) {
          const int s = step % C::kStages, ph = (step / C::kStages) & 1;
          const uint32_t bar = smem_u32(&bars->full[s]);
          const uint32_t dst = smem_base + s * C::kStageBytes;
          if (step < early) {  // first use of the stage: nothing to wait for, the barrier already expects the bytes
            tma_load_2d(dst, &a_map, bar, ks * kBK, mb * kBM);
            continue;
          }
          if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1)) { atomicCAS(status, 0u, 0x500u + s); ok = false; break; }
          mbar_arrive_expect_tx(bar, C::kStageBytes);
          tma_load_2d(dst, &a_map, bar, ks * kBK, mb * kBM);
          tma_load_2d(dst + kBM * kBK, &b_map, bar, 0, b_block_row(nb * BN, ks, ksteps));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(2, 1, 1, 0, 0, kBM, BN);  // s32 accumulators, s8 x s8, both K-major
      int step = 0, lt = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < ntiles; item += gridDim.x, ++lt) {
        const int kz = item % ksplit;
        const int ks0 = (int)((long long)kz * ksteps / ksplit), ks1 = (int)((long long)(kz + 1) * ksteps / ksplit);
        const int as = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&bars->acc_empty[as]), aph ^ 1)) { atomicCAS(status, 0u, 0x510u + as); break; }
        tc_fence_after();
        for (int ks = ks0; ks < ks1; ++ks, ++step) {
          const int s = step % C::kStages, ph = (step / C::kStages) & 1;
          if (!mbar_wait(smem_u32(&bars->full[s]), ph)) { atomicCAS(status, 0u, 0x520u + s); ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_base + s * C::kStageBytes, b_base = a_base + kBM * kBK;
#pragma unroll
          for (int j = 0; j < kBK / 32; ++j) {
            const uint64_t ad = umma_smem_desc_sw128(a_base + j * 32, 16, 1024);
            const uint64_t bd = umma_smem_desc_sw128(b_base + j * 32, 16, 1024);
            mma_i8_ss(tmem + as * BN, ad, bd, idesc, ((ks - ks0) | j) != 0);
          }
          mma_commit(smem_u32(&bars->empty[s]));
        }
        if (ok) mma_commit(smem_u32(&bars->acc_full[as]));
      }
    }
  } else {
    const int q = warp & 3;
    float* sb_s = reinterpret_cast<float*>(smem + C::kOffSb) + (warp - 2) * BN;
    int lt = 0;
    for (int item = blockIdx.x; item < ntiles; item += gridDim.x, ++lt) {
      const int tile = item / ksplit;
      const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
      const int as = lt & 1, aph = (lt >> 1) & 1;
      const int row = mb * kBM + q * 32 + lane;
      const bool row_ok = row < t;
      const float s_row = row_ok ? sa[row] : 0.f;
      __syncwarp();
      for (int i = lane; i < BN; i += 32) sb_s[i] = (nb * BN + i < n) ? sb[nb * BN + i] : 0.f;
      __syncwarp();
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_full[as]), aph))) { atomicCAS(status, 0u, 0x530u + as); break; }
      tc_fence_after();
      // scales, optional bias, 16-byte stores of one row's 32 columns (and the raw accumulators when asked for)
      auto emit = [&](const uint32_t (&v)[32], int c0) {
        const int col0 = nb * BN + c0;
        if (!(row_ok && col0 < n)) return;
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float f0 = ((float)(int)v[2 * j] * s_row) * sb_s[c0 + 2 * j];
          const float f1 = ((float)(int)v[2 * j + 1] * s_row) * sb_s[c0 + 2 * j + 1];
          w[j] = pack_out2<OutT>(f0, f1);
        }
        OutT* orow = out + (int64_t)row * n + col0;
        if (bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (col0 + 2 * j < n) {
              const float2 o = unpack_out2(w[j], OutT());
              const float2 b = unpack_out2(*reinterpret_cast<const uint32_t*>(bias + col0 + 2 * j), OutT());
              w[j] = pack_out2<OutT>(o.x + b.x, o.y + b.y);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (col0 + 8 * j < n) reinterpret_cast<uint4*>(orow)[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        if (acc_out != nullptr) {
          int32_t* arow = acc_out + (int64_t)row * n + col0;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (col0 + 4 * j < n) reinterpret_cast<uint4*>(arow)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
      };
      if (ksplit == 1) {
#pragma unroll 2
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + as * BN + c0, v);
          tmem_ld_wait();
          emit(v, c0);
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bars->acc_empty[as]));
    }
  }

  if (ksplit > 1) {
    // K-split (one work item per CTA, accumulator stage 0).  CTA `owner` of the cluster sums and writes rows
    // [owner * 128 / ksplit, ...) of the tile: every slice sends its int32 partial sums of those rows into slab
    // [slice] of the owner's shared memory, which reuses the operand stages.  Hence the first barrier: the epilogue
    // warps come here after their accumulator barrier, so past it every CTA's last MMA has read its operands.
    // Stores to a peer's shared memory do not wait for a round trip; the second barrier makes them visible, and
    // after it nobody touches another CTA's memory, so CTAs may leave independently.  Every thread of the cluster
    // passes both barriers (threads whose wait ran out included: the status word tells).  16-byte pieces are
    // XOR-swizzled by the row so that neither the stores (a lane per row) nor the reads (a warp per row) meet bank
    // conflicts.
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2) {
      // A lane holds one row of the accumulator, but a store to a peer should cover whole 128-byte lines: each
      // 32-column block is turned through a 4 KB staging area of the warp (behind the slabs), after which 8 lanes
      // send the 8 pieces of one line.  Staging and slabs use the same swizzle, so pieces are copied in place.
      const int q = warp & 3, rows_cta = kBM / ksplit;
      const uint32_t rank = cluster_cta_rank();
      uint4* stage = reinterpret_cast<uint4*>(smem + kBM * BN * 4) + (warp - 2) * 256;  // 32 rows x 8 pieces
      const int piece = lane & 7, sub = lane >> 3;
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) stage[lane * 8 + (j ^ (lane & 7))] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = q * 32 + i * 4 + sub;
          const uint32_t owner = (uint32_t)(r / rows_cta), rl = (uint32_t)(r % rows_cta);
          const uint4 u = stage[(i * 4 + sub) * 8 + piece];
          const uint32_t slab_piece = smem_base + (((rank * rows_cta + rl) * (BN / 4)) + (uint32_t)((c0 >> 2) + piece)) * 16u;
          st_cluster_shared_v4(cluster_map_shared(slab_piece, owner), u.x, u.y, u.z, u.w);
        }
        __syncwarp();
      }
      tc_fence_before();
    }
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2) {
      const int rank = (int)cluster_cta_rank(), tile = blockIdx.x / ksplit;
      const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
      const int rows_cta = kBM / ksplit;
      const float* sb_s = reinterpret_cast<float*>(smem + C::kOffSb) + (warp - 2) * BN;  // this warp's copy, filled above
      constexpr int kLanesPerRow = BN / 8, kRowsPerPass = 32 / kLanesPerRow;  // a warp covers 1, 2 or 4 rows at a time
      const int cl = lane % kLanesPerRow;
      const int col = nb * BN + 8 * cl;
      for (int rr = (warp - 2) * kRowsPerPass + lane / kLanesPerRow; rr < rows_cta; rr += 4 * kRowsPerPass) {
        const int r = rank * rows_cta + rr, row = mb * kBM + r;
        const uint32_t off0 = smem_base + (uint32_t)(rr * (BN / 4) + ((2 * cl) ^ (r & 7))) * 16u;
        const uint32_t off1 = smem_base + (uint32_t)(rr * (BN / 4) + ((2 * cl + 1) ^ (r & 7))) * 16u;
        const uint32_t slab = (uint32_t)(rows_cta * (BN / 4)) * 16u;
        uint32_t v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 8
        for (int z = 0; z < ksplit; ++z) {
          const uint4 p0 = ld_shared_v4(off0 + (uint32_t)z * slab);
          const uint4 p1 = ld_shared_v4(off1 + (uint32_t)z * slab);
          v[0] += p0.x; v[1] += p0.y; v[2] += p0.z; v[3] += p0.w;
          v[4] += p1.x; v[5] += p1.y; v[6] += p1.z; v[7] += p1.w;
        }
        if (row < t && col < n) {
          const float s_row = sa[row];
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            w[j] = pack_out2<OutT>(((float)(int)v[2 * j] * s_row) * sb_s[8 * cl + 2 * j],
                                   ((float)(int)v[2 * j + 1] * s_row) * sb_s[8 * cl + 2 * j + 1]);
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 o = unpack_out2(w[j], OutT());
              const float2 b = unpack_out2(*reinterpret_cast<const uint32_t*>(bias + col + 2 * j), OutT());
              w[j] = pack_out2<OutT>(o.x + b.x, o.y + b.y);
            }
          }
          *reinterpret_cast<uint4*>(out + (int64_t)row * n + col) = make_uint4(w[0], w[1], w[2], w[3]);
          if (acc_out != nullptr) {
            uint4* arow = reinterpret_cast<uint4*>(acc_out + (int64_t)row * n + col);
            arow[0] = make_uint4(v[0], v[1], v[2], v[3]);
            arow[1] = make_uint4(v[4], v[5], v[6], v[7]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// ---- 256 x 256 output tile per CTA: two 128-row accumulators share every B slice ------------------------------------
// A 128 x 256 tile needs 48 KB of operands per 512 tensor-core cycles; taking two row blocks against the same 256
// columns needs 64 KB per 1024 cycles, a third less per MMA, which is what the L2 -> shared-memory path can keep up
// with.  The two accumulators fill tensor memory (2 x 256 columns), so the epilogue of a tile does not overlap the
// next tile's main loop; sixteen epilogue warps (one per accumulator, lane quadrant and column half) keep it short.
constexpr int kDualThreads = 576;  // TMA, MMA issuer, 16 epilogue warps
struct DualCfg {
  static constexpr int kStageBytes = (2 * kBM + 256) * kBK;  // A rows 0-127, A rows 128-255, B
  static constexpr int kStages = 3;
  static constexpr int kOffSb = kStages * kStageBytes;       // 16 warps x 128 floats
  static constexpr int kOffBar = kOffSb + 16 * 128 * 4;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;
};

template <typename OutT>
__global__ void __launch_bounds__(kDualThreads, 1)
gemm_s8_dual_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                    const float* __restrict__ sa, const float* __restrict__ sb, OutT* __restrict__ out,
                    int32_t* __restrict__ acc_out, const OutT* __restrict__ bias, int t, int n, int k,
                    uint32_t* __restrict__ status) {
  using C = DualCfg;
  constexpr int BN = 256, BM2 = 2 * kBM;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmBars* bars = reinterpret_cast<GemmBars*>(smem + C::kOffBar);
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_n = (n + BN - 1) / BN, tiles_m = (t + BM2 - 1) / BM2;
  const int ntiles = tiles_m * tiles_n, ksteps = (k + kBK - 1) / kBK;

  if (tid == 0) {
    for (int i = 0; i < C::kStages; ++i) { mbar_init(smem_u32(&bars->full[i]), 1); mbar_init(smem_u32(&bars->empty[i]), 1); }
    mbar_init(smem_u32(&bars->acc_full[0]), 1);
    mbar_init(smem_u32(&bars->acc_empty[0]), 16);  // one arrival per epilogue warp
    fence_barrier_init();
    prefetch_tensormap(&a_map);
    prefetch_tensormap(&b_map);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int step = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
        const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
        for (int ks = 0; ks < ksteps; ++ks, ++step) {
          const int s = step % C::kStages, ph = (step / C::kStages) & 1;
          if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1)) { atomicCAS(status, 0u, 0x540u + s); ok = false; break; }
          const uint32_t bar = smem_u32(&bars->full[s]);
          mbar_arrive_expect_tx(bar, C::kStageBytes);
          const uint32_t dst = smem_base + s * C::kStageBytes;
          tma_load_2d(dst, &a_map, bar, ks * kBK, mb * BM2);
          tma_load_2d(dst + kBM * kBK, &a_map, bar, ks * kBK, mb * BM2 + kBM);
          tma_load_2d(dst + 2 * kBM * kBK, &b_map, bar, 0, b_block_row(nb * BN, ks, ksteps));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(2, 1, 1, 0, 0, kBM, BN);  // s32 accumulators, s8 x s8, both K-major
      int step = 0, lt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x, ++lt) {
        if (!mbar_wait(smem_u32(&bars->acc_empty[0]), (lt & 1) ^ 1)) { atomicCAS(status, 0u, 0x550u); break; }
        tc_fence_after();
        for (int ks = 0; ks < ksteps; ++ks, ++step) {
          const int s = step % C::kStages, ph = (step / C::kStages) & 1;
          if (!mbar_wait(smem_u32(&bars->full[s]), ph)) { atomicCAS(status, 0u, 0x560u + s); ok = false; break; }
          tc_fence_after();
          const uint32_t a0_base = smem_base + s * C::kStageBytes, a1_base = a0_base + kBM * kBK, b_base = a0_base + 2 * kBM * kBK;
#pragma unroll
          for (int j = 0; j < kBK / 32; ++j) {
            const uint64_t bd = umma_smem_desc_sw128(b_base + j * 32, 16, 1024);
            mma_i8_ss(tmem, umma_smem_desc_sw128(a0_base + j * 32, 16, 1024), bd, idesc, (ks | j) != 0);
            mma_i8_ss(tmem + BN, umma_smem_desc_sw128(a1_base + j * 32, 16, 1024), bd, idesc, (ks | j) != 0);
          }
          mma_commit(smem_u32(&bars->empty[s]));
        }
        if (ok) mma_commit(smem_u32(&bars->acc_full[0]));
      }
    }
  } else {
    const int q = warp & 3, half = ((warp - 2) >> 2) & 1, ch = (warp - 2) >> 3;  // lane quadrant, accumulator (row block), column half
    constexpr int kCols = BN / 2;
    float* sb_s = reinterpret_cast<float*>(smem + C::kOffSb) + (warp - 2) * kCols;
    int lt = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++lt) {
      const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
      const int row = mb * BM2 + half * kBM + q * 32 + lane;
      const bool row_ok = row < t;
      const float s_row = row_ok ? sa[row] : 0.f;
      __syncwarp();
      for (int i = lane; i < kCols; i += 32) sb_s[i] = (nb * BN + ch * kCols + i < n) ? sb[nb * BN + ch * kCols + i] : 0.f;
      __syncwarp();
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_full[0]), lt & 1))) { atomicCAS(status, 0u, 0x570u); break; }
      tc_fence_after();
#pragma unroll 2
      for (int cc = 0; cc < kCols; cc += 32) {
        const int c0 = ch * kCols + cc;
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + half * BN + c0, v);
        tmem_ld_wait();
        const int col0 = nb * BN + c0;
        if (row_ok && col0 < n) {
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float f0 = ((float)(int)v[2 * j] * s_row) * sb_s[cc + 2 * j];
            const float f1 = ((float)(int)v[2 * j + 1] * s_row) * sb_s[cc + 2 * j + 1];
            w[j] = pack_out2<OutT>(f0, f1);
          }
          OutT* orow = out + (int64_t)row * n + col0;
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (col0 + 2 * j < n) {
                const float2 o = unpack_out2(w[j], OutT());
                const float2 b = unpack_out2(*reinterpret_cast<const uint32_t*>(bias + col0 + 2 * j), OutT());
                w[j] = pack_out2<OutT>(o.x + b.x, o.y + b.y);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (col0 + 8 * j < n) reinterpret_cast<uint4*>(orow)[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          if (acc_out != nullptr) {
            int32_t* arow = acc_out + (int64_t)row * n + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col0 + 4 * j < n) reinterpret_cast<uint4*>(arow)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive_warp(smem_u32(&bars->acc_empty[0]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn gemm_encode_fn() {
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

int make_map_s8(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)k};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = gemm_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QO_ERR_CUDA, "int4_matmul: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return QO_OK;
}

// the blocked B operand as a matrix of 128-byte rows (256 per block); a box is one slice of box_rows channels
int make_map_b(CUtensorMap* map, const void* base, int64_t n, int64_t k, int box_rows) {
  const int64_t rows = ((n + 255) / 256) * ((k + kBK - 1) / kBK) * 256;
  const cuuint64_t dims[2] = {(cuuint64_t)kBK, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kBK};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = gemm_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QO_ERR_CUDA, "int4_matmul: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return QO_OK;
}

template <int BN, typename OutT>
int launch_gemm_tile(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out, int32_t* acc_out,
                     const void* bias, int64_t t, int64_t k, int64_t n, uint32_t* status, cudaStream_t stream, int ksplit = 1,
                     bool b_early = false) {
  using C = GemmCfg<BN>;
  CUtensorMap a_map, b_map;
  int rc = make_map_s8(&a_map, a8, t, k, kBM);
  if (rc) return rc;
  if ((rc = make_map_b(&b_map, b8, n, k, BN))) return rc;
  auto kern = gemm_s8_sm100_kernel<BN, OutT>;
  int dev = 0, sms = 148;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    QO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured[dev & 63] = true;
  }
  sms = sm_count(dev);
  const int64_t ntiles = ((t + kBM - 1) / kBM) * ((n + BN - 1) / BN) * ksplit;
  // K-split: one work item per CTA, the ksplit slices of a tile form a cluster
  const int grid = (int)((ksplit > 1 || ntiles < sms) ? ntiles : sms);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.numAttrs = 1;
  if (ksplit > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)ksplit;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  QO_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a_map, b_map, sa, sb, reinterpret_cast<OutT*>(out), acc_out,
                                 reinterpret_cast<const OutT*>(bias), (int)t, (int)n, (int)k, ksplit, b_early ? 1 : 0, status));
  return check_launch("gemm_s8_sm100_kernel");
}

}  // namespace

template <typename OutT>
int launch_gemm_dual(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out, int32_t* acc_out,
                     const void* bias, int64_t t, int64_t k, int64_t n, uint32_t* status, cudaStream_t stream) {
  CUtensorMap a_map, b_map;
  int rc = make_map_s8(&a_map, a8, t, k, kBM);
  if (rc) return rc;
  if ((rc = make_map_b(&b_map, b8, n, k, 256))) return rc;
  auto kern = gemm_s8_dual_kernel<OutT>;
  int dev = 0;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    QO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DualCfg::kSmemBytes));
    configured[dev & 63] = true;
  }
  const int sms = sm_count(dev);
  const int64_t ntiles = ((t + 2 * kBM - 1) / (2 * kBM)) * ((n + 255) / 256);
  const int grid = (int)(ntiles < sms ? ntiles : sms);
  kern<<<grid, kDualThreads, DualCfg::kSmemBytes, stream>>>(a_map, b_map, sa, sb, reinterpret_cast<OutT*>(out), acc_out,
                                                            reinterpret_cast<const OutT*>(bias), (int)t, (int)n, (int)k, status);
  return check_launch("gemm_s8_dual_kernel");
}

namespace {

// How many clusters of `size` CTAs of the K-split kernel with BN-wide tiles the device runs at once (0 if the query
// fails); cached.
template <int BN, typename OutT>
int max_split_clusters(int dev, int size) {
  static int cached[64][4] = {};  // [device][log2(size)], 0 = not asked yet, -1 = failed
  const int lg = size == 8 ? 3 : (size == 4 ? 2 : 1);
  int& c = cached[dev & 63][lg];
  if (c == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(size * 64));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = GemmCfg<BN>::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    (void)cudaFuncSetAttribute(gemm_s8_sm100_kernel<BN, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmemBytes);
    if (cudaOccupancyMaxActiveClusters(&n, gemm_s8_sm100_kernel<BN, OutT>, &cfg) != cudaSuccess) { (void)cudaGetLastError(); n = -1; }
    c = n > 0 ? n : -1;
  }
  return c > 0 ? c : 0;
}

// K slices per output tile of 128 x BN (1, 2, 4 or 8: the slices of a tile form a thread-block cluster).  Few tiles (a
// short activation matrix) leave most SMs idle and small tiles re-read the activations once per column tile, so the
// tiles stay wide and K is split instead.  All clusters of a launch should run at once (a second wave would double
// the time), so the split is lowered until the device says they do.
template <int BN, typename OutT>
int gemm_k_split(int dev, int64_t t, int64_t k, int64_t n) {
  if (n < BN) return 1;
  const int64_t tiles = ((t + kBM - 1) / kBM) * ((n + BN - 1) / BN), ksteps = (k + kBK - 1) / kBK;
  if (tiles >= 120) return 1;
  int64_t limit = 148 / tiles;
  if (limit > ksteps / 8) limit = ksteps / 8;
  int split = 1;
  while (split * 2 <= limit && split < 8) split *= 2;
  while (split > 1 && max_split_clusters<BN, OutT>(dev, split) < tiles) split /= 2;
  return split;
}

template <typename OutT>
int launch_gemm_typed(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out, int32_t* acc_out,
                      const void* bias, int64_t t, int64_t k, int64_t n, uint32_t* status, cudaStream_t stream,
                      bool b_early = false) {
  int dev = 0;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  const int ksplit = gemm_k_split<256, OutT>(dev, t, k, n);
  if (t <= kBM) {
    // one row block: tiles half as wide put twice as many CTAs to work when the wide ones leave half the SMs idle
    const int64_t ctas256 = ((n + 255) / 256) * ksplit;
    const int ksplit128 = gemm_k_split<128, OutT>(dev, t, k, n);
    const int64_t ctas128 = ((n + 127) / 128) * ksplit128;
    if (ksplit128 > 1 && ctas256 <= 74 && ctas128 > ctas256)
      return launch_gemm_tile<128, OutT>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream, ksplit128, b_early);
  }
  if (ksplit > 1)
    return launch_gemm_tile<256, OutT>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream, ksplit, b_early);
  // enough 256 x 256 tiles to keep the CTA pairs busy, and a row count that the 256-row tiles do not pad by much:
  // the CTA-pair kernel (each CTA stages half of B, a third less shared-memory traffic per MMA)
  {
    const int64_t tiles_pair = ((t + 2 * kBM - 1) / (2 * kBM)) * ((n + 255) / 256);
    const int64_t rows256 = ((t + 255) / 256) * 256, rows128 = ((t + 127) / 128) * 128;
    if (current_kernel_policy() != 3 && n >= 256 && tiles_pair >= 48 && rows256 * 8 <= rows128 * 9) {
      const int rc = launch_gemm_sm100_pair(a8, b8, sa, sb, out, std::is_same<OutT, __half>::value ? QO_F16 : QO_BF16, t, k, n,
                                            acc_out, bias, status, stream);
      if (rc != QO_ERR_UNSUPPORTED) return rc;
    }
  }
  // enough 256 x 256 tiles for every SM: two accumulators per CTA share each B slice
  // (with few tiles and a short K the unshared tile does better: its epilogue overlaps the next main loop and its
  // smaller tiles fill the last wave more evenly)
  const int64_t tiles2 = ((t + 2 * kBM - 1) / (2 * kBM)) * ((n + 255) / 256);
  if (n >= 256 && tiles2 >= 140 && (k >= 8192 || tiles2 >= 4 * 148))
    return launch_gemm_dual<OutT>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream);
  // widest tile that does not leave most SMs idle
  const int64_t tiles_m = (t + kBM - 1) / kBM;
  if (n >= 256 && tiles_m * ((n + 255) / 256) >= 120)
    return launch_gemm_tile<256, OutT>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream, 1, b_early);
  if (n >= 128 && tiles_m * ((n + 127) / 128) >= 100)
    return launch_gemm_tile<128, OutT>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream, 1, b_early);
  return launch_gemm_tile<64, OutT>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream, 1, b_early);
}

inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

// bytes of the blocked int8 B operand: whole blocks of 256 channels x 128 K-bytes
size_t gemm_b8_bytes(int64_t n, int64_t k) {
  if (n <= 0 || k <= 0) return 0;
  return (size_t)((n + 255) / 256) * (size_t)((k + kBK - 1) / kBK) * (size_t)(256 * kBK);
}

size_t gemm_sm100_workspace_bytes(int64_t t, int64_t k, int64_t n) {
  if (t <= 0 || k <= 0 || n <= 0) return 0;
  return align256((size_t)t * k) + gemm_b8_bytes(n, k);
}

bool gemm_sm100_supported(int64_t t, int64_t k, int64_t n, int64_t lda, int64_t bsk, int64_t bsn) {
  (void)lda;
  if (k % 16 || k < 16) return false;              // TMA: row stride of the widened operands must be 16-byte aligned
  if (n % 8) return false;                         // 16-byte output stores
  if (t > 0x7fffff00LL || n > 0x7fffff00LL || k > 262143) return false;
  if (((n + 255) / 256) * ((k + kBK - 1) / kBK) * 256 > 0x7fffff00LL) return false;  // 128-byte rows of the blocked B operand (TMA coordinate)
  if (bsk != 1 && bsn != 1) return false;
  return gemm_encode_fn() != nullptr;
}

int launch_gemm_sm100_s8(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out, int out_dtype,
                         int64_t t, int64_t k, int64_t n, int32_t* acc_out, const void* bias, cudaStream_t stream, bool b_early) {
  if (reinterpret_cast<uintptr_t>(a8) % 16 || reinterpret_cast<uintptr_t>(b8) % 16 || reinterpret_cast<uintptr_t>(out) % 16 ||
      (acc_out && reinterpret_cast<uintptr_t>(acc_out) % 16) || (bias && reinterpret_cast<uintptr_t>(bias) % 4))
    return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: operands of the tcgen05 kernel must be 16-byte aligned");
  int dev = 0;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  uint32_t* status = device_status_word(dev);
  if (!status) return fail(QO_ERR_CUDA, "int4_matmul: could not allocate the device status word");
  if (out_dtype == QO_F16) return launch_gemm_typed<__half>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream, b_early);
  if (out_dtype == QO_BF16) return launch_gemm_typed<__nv_bfloat16>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream, b_early);
  return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: out_dtype must be QO_F16 or QO_BF16");
}

// blocked: write the layout of the B operand (see the head of this file) instead of row-major
// beside_previous: neither `in` nor `out` is touched by the kernel that precedes this one in the stream, and that
// kernel releases its dependents only after its own dependency wait (the quantizers do): the pass may run beside it
int launch_widen_rows(const int32_t* in, int64_t ld_words, int8_t* out, int64_t rows, int64_t k, cudaStream_t stream, bool blocked,
                      bool beside_previous) {
  const int64_t ksteps = blocked ? (k + kBK - 1) / kBK : 0;
  if ((k % 32) == 0 && (ld_words % 4) == 0 && reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    const WidenJob job = {reinterpret_cast<const uint32_t*>(in), reinterpret_cast<uint8_t*>(out), ld_words, rows, k / 32, ksteps};
    const WidenJob none = {nullptr, nullptr, 0, 0, 1, 0};
    int64_t blocks = (rows * (k / 32) + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (blocks < 1) blocks = 1;
    if (beside_previous) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)blocks);
      cfg.blockDim = dim3(256);
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      QO_CUDA_TRY(cudaLaunchKernelEx(&cfg, widen_rows2_kernel, job, none, 1));
    } else {
      widen_rows2_kernel<<<(int)blocks, 256, 0, stream>>>(job, none, 0);
    }
    return check_launch("widen_rows2_kernel");
  }
  const int64_t total = rows * (k / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  widen_rows_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(in), ld_words,
                                                     reinterpret_cast<uint8_t*>(out), rows, k / 8, ksteps);
  return check_launch("widen_rows_kernel");
}

int launch_gemm_sm100(const int32_t* a, int64_t lda, const int32_t* b, int64_t bsk, int64_t bsn, const float* sa,
                      const float* sb, void* out, int out_dtype, int64_t t, int64_t k, int64_t n, int32_t* acc_out,
                      const void* bias, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (workspace_bytes < gemm_sm100_workspace_bytes(t, k, n) || reinterpret_cast<uintptr_t>(workspace) % 256)
    return fail(QO_ERR_WORKSPACE, "int4_matmul: workspace missing, too small or not 256-byte aligned");
  int rc;
  // prefill-sized products with K-contiguous operands: the kernel that unpacks the nibbles itself (no widening pass,
  // the workspace stays untouched)
  if (gemm_unpack_supported(t, k, n, a, lda, b, bsk, bsn) && gemm_unpack_preferred(t, k, n)) {
    int dev = 0;
    QO_CUDA_TRY(cudaGetDevice(&dev));
    uint32_t* status = device_status_word(dev);
    if (!status) return fail(QO_ERR_CUDA, "int4_matmul: could not allocate the device status word");
    rc = launch_gemm_unpack(a, lda, b, bsn, sa, sb, out, out_dtype, t, k, n, acc_out, bias, status, stream);
    if (rc != QO_ERR_UNSUPPORTED) return rc;
  }
  int8_t* a8 = reinterpret_cast<int8_t*>(workspace);
  int8_t* b8 = a8 + align256((size_t)t * k);
  if (bsk == 1 && (k % 32) == 0 && (lda % 4) == 0 && (bsn % 4) == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(b) % 16 == 0) {
    // both operands have K contiguous and 16-byte aligned rows: one launch widens both
    const WidenJob ja = {reinterpret_cast<const uint32_t*>(a), reinterpret_cast<uint8_t*>(a8), lda, t, k / 32, 0};
    const WidenJob jb = {reinterpret_cast<const uint32_t*>(b), reinterpret_cast<uint8_t*>(b8), bsn, n, k / 32, (k + kBK - 1) / kBK};
    const int64_t total = (t + n) * (k / 32);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    widen_rows2_kernel<<<(int)blocks, 256, 0, stream>>>(ja, jb, 0);
    if ((rc = check_launch("widen_rows2_kernel"))) return rc;
    return launch_gemm_sm100_s8(a8, b8, sa, sb, out, out_dtype, t, k, n, acc_out, bias, stream);
  }
  rc = launch_widen_rows(a, lda, a8, t, k, stream, false, false);
  if (rc) return rc;
  if (bsk == 1) {
    rc = launch_widen_rows(b, bsn, b8, n, k, stream, true, false);  // rows of the weight matrix [Nout, K/8]
  } else {
    dim3 grid((unsigned)((n + 31) / 32), (unsigned)((k / 8 + 31) / 32));
    widen_transpose_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(b), bsk, bsn,
                                                     reinterpret_cast<uint8_t*>(b8), n, k / 8, (k + kBK - 1) / kBK);
    rc = check_launch("widen_transpose_kernel");
  }
  if (rc) return rc;
  return launch_gemm_sm100_s8(a8, b8, sa, sb, out, out_dtype, t, k, n, acc_out, bias, stream);
}

// ---- pieces for callers that bring their own scratch and status word (int4_gemm_static.cu) ------------------------
int launch_widen_b(const int32_t* b, int64_t bsk, int64_t bsn, int8_t* b8, int64_t n, int64_t k, cudaStream_t stream) {
  if (bsk == 1) return launch_widen_rows(b, bsn, b8, n, k, stream, true, false);
  dim3 grid((unsigned)((n + 31) / 32), (unsigned)((k / 8 + 31) / 32));
  widen_transpose_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(b), bsk, bsn,
                                                   reinterpret_cast<uint8_t*>(b8), n, k / 8, (k + kBK - 1) / kBK);
  return check_launch("widen_transpose_kernel");
}

int launch_gemm_sm100_s8_status(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out,
                                int out_dtype, int64_t t, int64_t k, int64_t n, int32_t* acc_out, uint32_t* status,
                                cudaStream_t stream) {
  if (reinterpret_cast<uintptr_t>(a8) % 16 || reinterpret_cast<uintptr_t>(b8) % 16 || reinterpret_cast<uintptr_t>(out) % 16 ||
      (acc_out && reinterpret_cast<uintptr_t>(acc_out) % 16))
    return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: operands of the tcgen05 kernel must be 16-byte aligned");
  if (out_dtype == QO_F16) return launch_gemm_typed<__half>(a8, b8, sa, sb, out, acc_out, nullptr, t, k, n, status, stream);
  if (out_dtype == QO_BF16) return launch_gemm_typed<__nv_bfloat16>(a8, b8, sa, sb, out, acc_out, nullptr, t, k, n, status, stream);
  return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: out_dtype must be QO_F16 or QO_BF16");
}

}  // namespace qo
