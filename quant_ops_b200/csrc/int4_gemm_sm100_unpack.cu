// Packed-int4 GEMM for sm_100a with the nibbles unpacked INSIDE the kernel: no widening pass, no workspace.
//
// TMA brings PACKED tiles of both operands into shared memory (128 bytes = 256 int4 values per row and stage, 128-byte
// swizzle), converter warps turn the nibbles into int8 operands, tcgen05.mma kind::i8 accumulates in int32 in tensor
// memory, and the epilogue applies (float(acc) * scale_a[row]) * scale_b[col] -- the arithmetic of the reference kernel
// (src/quant_ops/ops/quantization/int4_matmul/kernels/cuda_int4_matmul_kernel.cu:81-116, which also unpacks on its
// load path).  The work is laid out for CTA pairs (cta_group::2): two CTAs on the SMs of one TPC share a 256 x 256
// output tile; each CTA owns 128 rows of A and 128 of the tile's B rows.
//
// What shaped the kernel (cycle counts measured on B200 with a single issuing thread, K = 32 per MMA):
//   * An MMA whose A operand comes from TENSOR MEMORY runs at the tensor pipe's nominal rate (M = 256, N = 256 over a
//     pair: 138 cycles), one whose A comes from shared memory needs 173: A's packed rows are therefore read once by
//     converter warps (one thread per row), widened in registers and written to tensor memory (tcgen05.st); only B
//     becomes an int8 tile in shared memory (128-byte swizzle), written by a second group of converter warps.
//   * Every tcgen05.commit costs the issuing thread about 60 cycles during which it issues no MMA, and the peer CTA
//     needs its own: a stage therefore carries 256 values of K (eight MMAs per pair of commits).
//   * A barrier probe answers after about 200 cycles even when the phase is long complete: the issuing thread probes
//     the NEXT stage's barrier before it issues the MMAs of this one and looks at the answer afterwards.
//   * A TMA load of a 32 KB stage takes about 1400 cycles from request to arrival (operands in L2), longer than a
//     stage's MMAs (about 1100): the packed ring is three stages deep, as is the operand ring behind it.
//   * Tensor memory (512 columns) holds ONE 256-column accumulator and three A stages of 64 columns; the epilogue (8
//     warps) therefore does not overlap the next tile's main loop, but frees the accumulator as soon as its last
//     values are in registers.
//
// Unpacking without sign extension: x ^ 0x88888888 turns the offset-binary nibbles into two's-complement nibbles, and a
// nibble in the HIGH half of a byte is the int8 value 16 * n.  Each packed word yields one word of its even elements
// ((t << 4) & 0xF0F0F0F0) and one of its odd elements (t & 0xF0F0F0F0); both operands use the same (permuted) order
// of K, a dot product does not care, and every product carries the factor 256, which an arithmetic shift removes
// exactly in the epilogue (|256 * acc| < 2^31 for K <= 131072).  Four integer instructions per eight values.
//
// Roles (28 warps per CTA; both CTAs of a pair run the same code, only the leader issues MMAs):
//   warp 0       TMA producer: packed A block + packed B half into a ring of 3 stages (local barriers)
//   warp 1       leader: tcgen05.mma.cta_group::2, M = 256, N = 256, eight K = 32 slices per stage; commits release the
//                operand stage in BOTH CTAs (one commit per CTA, the peer's barrier addressed through mapa)
//   warps 2-9    epilogue of the CTA's own 128 accumulator rows (two warps per lane quadrant, 128 columns each)
//   warps 10-21  A converters: three sets of four warps, set g takes the stages g, g + 3, ...; thread = row, lane
//                quadrant = warp % 4
//   warps 22-27  B converters: three sets of two warps, same rotation
//   Converters of both CTAs report to the leader's "operands ready" barrier (remote arrivals from the peer).
//   A converter's work per stage is a chain of fixed latencies (barrier poll, shared-memory loads, the tensor-memory
//   or shared-memory stores, a proxy fence, the arrival); sets in rotation keep one chain per set off the critical
//   path.  There are as many sets as ring slots, so a set always works on the same slot and sees EVERY phase of the
//   barriers it waits on.  That is required, not a nicety: a parity wait cannot tell use u of a slot from use u - 2, and
//   TMA loads complete out of order (a box that lies outside the tensor is filled at once), so a set that visited a
//   slot on every second use only was measured to pass a wait one use early and to release the slot under its readers.
//
// Every mbarrier wait is bounded; a wait that runs out records a code in the device status word and its role leaves.
// The cluster barriers at set-up and tear-down are hardware barriers that every thread of both CTAs reaches.
#include <mutex>

#include "qo_internal.cuh"
#include "sm100_ptx.cuh"

namespace qo {
namespace {

using namespace ptx;

constexpr int kBM = 128;        // rows per CTA
constexpr int kBN = 256;        // columns of the pair's tile
constexpr int kBNh = kBN / 2;   // B rows staged per CTA
constexpr int kKStage = 256;    // int4 values per stage = 128 packed bytes = 256 int8 bytes per row
constexpr int kSets = 3;        // converter sets in rotation = ring depth: set g always works on slot g of both rings
constexpr int kThreads = 28 * 32;
constexpr int kPStages = kSets;     // packed ring
constexpr int kOStages = kSets;     // operand ring (int8 B in shared memory, A in tensor memory)
constexpr int kPABytes = kBM * 128, kPBBytes = kBNh * 128, kPStageBytes = kPABytes + kPBBytes;  // 16 KB + 16 KB
constexpr int kOAtomBytes = kBNh * 128;                 // one 128-byte K atom of the int8 B half: 16 KB
constexpr int kOBBytes = 2 * kOAtomBytes;               // 32 KB per operand stage
constexpr int kOffP = 0;
constexpr int kOffO = kOffP + kPStages * kPStageBytes;  // 96 KB
constexpr int kOffSb = kOffO + kOStages * kOBBytes;     // +96 KB; 8 epilogue warps x 128 floats
constexpr int kOffBar = kOffSb + 8 * 128 * 4;
constexpr int kSmemBytes = kOffBar + 512 + 1024;
constexpr int kColA = kBN;      // first tensor-memory column of the A operand stages (64 columns each)
constexpr int kEpiWarp0 = 2, kAWarp0 = 10, kBWarp0 = 22;

struct Bars {
  uint64_t p_full[kPStages], p_empty[kPStages];
  uint64_t op_ready[kOStages], op_empty[kOStages];
  uint64_t acc_full, acc_empty;
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
__device__ __forceinline__ float2 unpack_out2(uint32_t w, __half) { return __half22float2(*reinterpret_cast<__half2*>(&w)); }
__device__ __forceinline__ float2 unpack_out2(uint32_t w, __nv_bfloat16) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w)); }

// packed word -> (even elements, odd elements) as int8 bytes holding 16 * value
__device__ __forceinline__ void split16(uint32_t w, uint32_t& even, uint32_t& odd) {
  // the shift as an integer multiply-add (FMA pipe), the mask and the sign flip of each operand as one three-input
  // logic operation (ALU pipe): two ALU instructions per packed word instead of three
  uint32_t w16;
  asm("mad.lo.u32 %0, %1, 16, 0;" : "=r"(w16) : "r"(w));
  asm("lop3.b32 %0, %1, 0xF0F0F0F0, 0x80808080, 0x6A;" : "=r"(even) : "r"(w16));  // (a & b) ^ c
  asm("lop3.b32 %0, %1, 0xF0F0F0F0, 0x80808080, 0x6A;" : "=r"(odd) : "r"(w));
}

// One stage of the leader's issue loop as a single instruction sequence: probe the NEXT stage's "operands ready"
// barrier, issue the eight K = 32 MMAs of this stage (A from tensor memory, 8 columns per slice; B descriptor advanced
// by 32 bytes per slice inside a 128-byte K atom, the second atom `atom_units` 16-byte units further), commit to the
// "stage free" barriers of both CTAs, and only then look at the probe's answer.  A warp issues in order and stalls at
// the first instruction that needs an outstanding result, so the probe only overlaps the MMAs if nothing between them
// reads its predicate.
__device__ __forceinline__ bool issue_stage(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                            uint32_t bar_free, uint32_t bar_free_peer, uint32_t bar_next, uint32_t parity_next) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred pn, pa;\n\t"
      ".reg .b32 a1, a2, a3, a4, a5, a6, a7;\n\t"
      ".reg .b64 b1, b2, b3, b4, b5, b6, b7;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 pn, [%8], %9;\n\t"
      "setp.ne.b32 pa, %5, 0;\n\t"
      "add.u32 a1, %2, 8;\n\t"
      "add.u32 a2, %2, 16;\n\t"
      "add.u32 a3, %2, 24;\n\t"
      "add.u32 a4, %2, 32;\n\t"
      "add.u32 a5, %2, 40;\n\t"
      "add.u32 a6, %2, 48;\n\t"
      "add.u32 a7, %2, 56;\n\t"
      "add.u64 b1, %3, 2;\n\t"
      "add.u64 b2, %3, 4;\n\t"
      "add.u64 b3, %3, 6;\n\t"
      "add.u64 b4, %3, %10;\n\t"
      "add.u64 b5, b4, 2;\n\t"
      "add.u64 b6, b4, 4;\n\t"
      "add.u64 b7, b4, 6;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%1], [%2], %3, %4, pa;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%1], [a1], b1, %4, 1;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%1], [a2], b2, %4, 1;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%1], [a3], b3, %4, 1;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%1], [a4], b4, %4, 1;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%1], [a5], b5, %4, 1;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%1], [a6], b6, %4, 1;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%1], [a7], b7, %4, 1;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t"
      "selp.u32 %0, 1, 0, pn;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(bar_free), "r"(bar_free_peer), "r"(bar_next),
        "r"(parity_next), "l"((uint64_t)(kOAtomBytes >> 4))
      : "memory");
  return ok != 0;
}

// GATHER: the outputs are not stored to `out` but, at row `row_offset + row`, into every buffer of `dsts` -- this GPU's
// own copy of the gathered output and the peers' copies, mapped into this process (plain stores over NVLink; the
// all-gather of a row-sharded layer's outputs costs no kernel of its own and no SMs).
template <typename OutT, bool GATHER>
__global__ void __launch_bounds__(kThreads, 1)
gemm_s4_unpack_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                      const float* __restrict__ sa, const float* __restrict__ sb, OutT* __restrict__ out,
                      int32_t* __restrict__ acc_out, const OutT* __restrict__ bias, int t, int n, int k, int items, int cut_from,
                      uint32_t* __restrict__ status, const __grid_constant__ GatherDsts dsts) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + kOffBar);
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tiles_n = (n + kBN - 1) / kBN;
  const int ksteps = k / kKStage;  // k is a multiple of 256 (checked by the host)
  // Work items: whole tiles, except that the tiles of a last wave which would occupy at most half of the pairs are cut
  // into two halves of 128 columns (MMAs with N = 128), so that twice as many pairs share that wave: 256 tiles on 74
  // pairs take the time of 3.7 tiles instead of 4.
  // (items and cut_from, the first item that is a half, come from the host: kernel parameters cost no registers)
  int mine = 0;                              // items of this pair
  if (pair < items) mine = (items - pair + npairs - 1) / npairs;
  const int total_steps = mine * ksteps;
  // item -> tile index, first column of the item inside the tile (0 or 128), columns of the item (256 or 128)
  auto item_of = [&](int item, int& tile, int& col_in_tile, int& width) {
    if (item < cut_from) { tile = item; col_in_tile = 0; width = kBN; }
    else { tile = cut_from + ((item - cut_from) >> 1); col_in_tile = ((item - cut_from) & 1) * (kBN / 2); width = kBN / 2; }
  };

  if (tid == 0) {
    for (int i = 0; i < kPStages; ++i) { mbar_init(smem_u32(&bars->p_full[i]), 1); mbar_init(smem_u32(&bars->p_empty[i]), 6); }
    for (int i = 0; i < kOStages; ++i) { mbar_init(smem_u32(&bars->op_ready[i]), 12); mbar_init(smem_u32(&bars->op_empty[i]), 1); }
    mbar_init(smem_u32(&bars->acc_full), 1);
    mbar_init(smem_u32(&bars->acc_empty), 16);
    fence_barrier_init();
    prefetch_tensormap(&a_map);
    prefetch_tensormap(&b_map);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();  // both CTAs' barriers and tensor memory exist before either touches the other
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  // Launched with programmatic stream serialization: everything above may overlap the tail of the preceding kernel.
  grid_dependency_wait();

  if (warp == 0) {
    // ---- TMA producer -------------------------------------------------------------------------------------------
    if (lane == 0) {
      int step = 0;
      bool ok = true;
      for (int item = pair; ok && item < items; item += npairs) {
        int tile, col_in_tile, width;
        item_of(item, tile, col_in_tile, width);
        const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
        // a CTA stages its half of the item's B rows; the box always has 128 rows, of which a half item uses the first 64
        const int row_a = mb * 2 * kBM + (int)rank * kBM, row_b = nb * kBN + col_in_tile + (int)rank * (width >> 1);
        for (int ks = 0; ks < ksteps; ++ks, ++step) {
          const int ps = step % kPStages, pph = (step / kPStages) & 1;
          if (!mbar_wait(smem_u32(&bars->p_empty[ps]), pph ^ 1)) { atomicCAS(status, 0u, 0xA00u + ps); ok = false; break; }
          const uint32_t bar = smem_u32(&bars->p_full[ps]);
          mbar_arrive_expect_tx(bar, kPStageBytes);
          const uint32_t dst = smem_base + kOffP + ps * kPStageBytes;
          tma_load_2d(dst, &a_map, bar, ks * 128, row_a);
          tma_load_2d(dst + kPABytes, &b_map, bar, ks * 128, row_b);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (leader CTA only) ----------------------------------------------------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_whole = umma_idesc(2, 1, 1, 0, 0, 2 * kBM, kBN);  // s32 accumulators, s8 x s8, K-major, M = 256 over the pair
      const uint32_t idesc_half = umma_idesc(2, 1, 1, 0, 0, 2 * kBM, kBN / 2);
      // one thread feeds the tensor cores of both SMs, so its instruction count per MMA matters: the B descriptor is
      // built once and advanced by adding to its address field (units of 16 bytes)
      const uint64_t b_desc0 = umma_smem_desc_sw128(smem_base + kOffO, 16, 1024);
      const uint32_t op_empty0 = smem_u32(&bars->op_empty[0]), op_empty0_peer = cluster_map_shared(op_empty0, 1);
      const uint32_t acc_full = smem_u32(&bars->acc_full), acc_full_peer = cluster_map_shared(acc_full, 1);
      int step = 0;
      bool ok = true, ready = false;  // ready: the operands of `step` were already seen complete by an early probe
      for (int lt = 0; ok && lt < mine; ++lt) {
        if (!mbar_wait(smem_u32(&bars->acc_empty), (lt & 1) ^ 1)) { atomicCAS(status, 0u, 0xA10u); break; }
        const uint32_t idesc = pair + lt * npairs >= cut_from ? idesc_half : idesc_whole;
        for (int ks = 0; ks < ksteps; ++ks, ++step) {
          const int s = step % kOStages, ph = (step / kOStages) & 1;
          if (!ready && !mbar_wait(smem_u32(&bars->op_ready[s]), ph)) { atomicCAS(status, 0u, 0xA20u + s); ok = false; break; }
          // the next stage's barrier is probed inside issue_stage, under this stage's MMAs (the last stage probes its
          // own, completed barrier: a harmless answer that is not used)
          const bool last = step + 1 >= total_steps;
          const int sn = last ? s : (step + 1) % kOStages, phn = last ? ph : ((step + 1) / kOStages) & 1;
          tc_fence_after();
          ready = issue_stage(tmem, tmem + kColA + s * 64, b_desc0 + (uint64_t)(s * (kOBBytes >> 4)), idesc, ks != 0,
                              op_empty0 + s * 8, op_empty0_peer + s * 8, smem_u32(&bars->op_ready[sn]), phn) && !last;
        }
        if (ok) {
          mma_commit_pair(acc_full);
          mma_commit_pair(acc_full_peer);
        }
      }
    }
  } else if (warp < kAWarp0) {
    // ---- epilogue: the CTA's own 128 rows of the tile; warp (q, half) takes columns 128 half .. of lanes 32 q .. ------
    const int q = warp & 3, half = (warp - kEpiWarp0) >> 2;
    const bool wide_stores = (n % 16) == 0 && (reinterpret_cast<uintptr_t>(out) % 32) == 0;  // rows start on 32-byte boundaries
    float* sb_s = reinterpret_cast<float*>(smem + kOffSb) + (warp - kEpiWarp0) * 128;
    for (int lt = 0; lt < mine; ++lt) {
      int tile, col_in_tile, width;
      item_of(pair + lt * npairs, tile, col_in_tile, width);
      const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
      const int wcols = width >> 1;  // columns of this warp: 128, or 64 of a half item
      const int row = mb * 2 * kBM + (int)rank * kBM + q * 32 + lane;
      const bool row_ok = row < t;
      // Both operands carried the factor 16.  float(256 * acc) is exact (|acc| < 2^23) and scaling by a power of two
      // commutes with rounding, so the factor is taken out of the row scale instead of out of every accumulator.
      const float s_row = row_ok ? sa[row] * 0.00390625f : 0.f;
      const int colw = nb * kBN + col_in_tile + half * wcols;  // first column of this warp
      __syncwarp();
      for (int i = lane; i < wcols; i += 32) sb_s[i] = (colw + i < n) ? sb[colw + i] : 0.f;
      __syncwarp();
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_full), lt & 1))) { atomicCAS(status, 0u, 0xA30u); break; }
      tc_fence_after();
#pragma unroll 1
      for (int cc = 0; cc < wcols; cc += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + half * wcols + cc, v);
        tmem_ld_wait();
        if (cc + 32 == wcols) {
          // the last accumulator values of this warp are in registers: the next tile's MMAs may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            const uint32_t e = smem_u32(&bars->acc_empty);
            if (rank == 0) mbar_arrive(e); else mbar_arrive_cluster(cluster_map_shared(e, 0));
          }
        }
        const int col0 = colw + cc;
        if (row_ok && col0 < n) {
          const int64_t off = (int64_t)(GATHER ? row + dsts.row_offset : row) * n + col0;
          // 16 columns at a time: eight packed words live beside the 32 accumulators, not sixteen
#pragma unroll
          for (int jh = 0; jh < 2; ++jh) {
            if (col0 + 16 * jh >= n) break;
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float4 sc = *reinterpret_cast<const float4*>(sb_s + cc + 16 * jh + 4 * j);
              const uint32_t* vv = v + 16 * jh + 4 * j;
              w[2 * j] = pack_out2<OutT>(((float)(int)vv[0] * s_row) * sc.x, ((float)(int)vv[1] * s_row) * sc.y);
              w[2 * j + 1] = pack_out2<OutT>(((float)(int)vv[2] * s_row) * sc.z, ((float)(int)vv[3] * s_row) * sc.w);
            }
            if (bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (col0 + 16 * jh + 2 * j < n) {
                  const float2 o = unpack_out2(w[j], OutT());
                  const float2 bb = unpack_out2(*reinterpret_cast<const uint32_t*>(bias + col0 + 16 * jh + 2 * j), OutT());
                  w[j] = pack_out2<OutT>(o.x + bb.x, o.y + bb.y);
                }
              }
            }
            // A lane owns a row, so a warp's store instruction touches 32 different lines; the exposed part of the
            // epilogue is bound by those line accesses.  32-byte stores (whole sectors) halve their number.
            if (GATHER) {
              // (the host admits only row lengths and buffers that make every piece a whole 32-byte sector)
              for (int d = 0; d < dsts.n_dst; ++d)
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(reinterpret_cast<OutT*>(dsts.ptr[d]) + off + 16 * jh),
                             "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
            } else if (wide_stores) {
              asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(out + off + 16 * jh), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                           "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
            } else {
              reinterpret_cast<uint4*>(out + off + 16 * jh)[0] = make_uint4(w[0], w[1], w[2], w[3]);
              if (col0 + 16 * jh + 8 < n) reinterpret_cast<uint4*>(out + off + 16 * jh)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          }
          if (acc_out != nullptr) {
            int32_t* arow = acc_out + (int64_t)row * n + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col0 + 4 * j < n)
                reinterpret_cast<uint4*>(arow)[j] = make_uint4((uint32_t)((int)v[4 * j] >> 8), (uint32_t)((int)v[4 * j + 1] >> 8),
                                                               (uint32_t)((int)v[4 * j + 2] >> 8), (uint32_t)((int)v[4 * j + 3] >> 8));
          }
        }
        __syncwarp();
      }
    }
  } else if (warp < kBWarp0) {
    // ---- A converters: set e takes the stages e, e + 3, ...; thread = one row of the CTA's A block ---------------------
    const int e = (warp - kAWarp0) >> 2, q = warp & 3, r = q * 32 + lane;  // set 0 .. 2
    const uint32_t row_off = (uint32_t)(r * 128), sw = (uint32_t)(r & 7);
    for (int step = e; step < total_steps; step += kSets) {
      const int ps = step % kPStages, pph = (step / kPStages) & 1;
      const int s = step % kOStages, ph = (step / kOStages) & 1;
      if (__any_sync(0xffffffffu, mbar_wait2(smem_u32(&bars->p_full[ps]), pph, smem_u32(&bars->op_empty[s]), ph ^ 1) != 0)) {
        atomicCAS(status, 0u, 0xA40u + ps);
        break;
      }
      tc_fence_after();
      const uint32_t src = smem_base + kOffP + ps * kPStageBytes + row_off;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint4 p[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) p[c] = ld_shared_v4(src + (((uint32_t)(4 * h + c) ^ sw) << 4));
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          split16(p[c].x, v[8 * c + 0], v[8 * c + 1]);
          split16(p[c].y, v[8 * c + 2], v[8 * c + 3]);
          split16(p[c].z, v[8 * c + 4], v[8 * c + 5]);
          split16(p[c].w, v[8 * c + 6], v[8 * c + 7]);
        }
        tmem_st_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + kColA + s * 64 + h * 32, v);
      }
      // The packed stage is released only here, after instructions that consume every loaded value: an arrival placed
      // right behind the ld.shared instructions was measured to let the next TMA overwrite rows that some lanes had
      // not read yet (nothing orders another lane's outstanding loads before lane 0's arrival).
      mbar_arrive_warp(smem_u32(&bars->p_empty[ps]));
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        const uint32_t ready = smem_u32(&bars->op_ready[s]);
        if (rank == 0) mbar_arrive(ready); else mbar_arrive_cluster(cluster_map_shared(ready, 0));
      }
    }
  } else {
    // ---- B converters: 128 rows x 8 packed 16-byte pieces per stage, sixteen per thread of the set on duty; eight
    // consecutive lanes take eight consecutive rows of one piece, which is conflict-free for the 128-byte-swizzled
    // reads and writes ---------------------------------------------------------------------------------------------
    const int f = (warp - kBWarp0) >> 1, bt = ((warp - kBWarp0) & 1) * 32 + lane;  // set 0 .. 2, thread within the set (0 .. 63)
    for (int step = f; step < total_steps; step += kSets) {
      const int ps = step % kPStages, pph = (step / kPStages) & 1;
      const int s = step % kOStages, ph = (step / kOStages) & 1;
      if (__any_sync(0xffffffffu, mbar_wait2(smem_u32(&bars->p_full[ps]), pph, smem_u32(&bars->op_empty[s]), ph ^ 1) != 0)) {
        atomicCAS(status, 0u, 0xA50u + ps);
        break;
      }
      const uint32_t src = smem_base + kOffP + ps * kPStageBytes + kPABytes;
      const uint32_t dst = smem_base + kOffO + s * kOBBytes;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 p[4];
        int rr[4], cc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int task = (g * 4 + i) * 64 + bt;  // 0 .. 1023
          cc[i] = task >> 7;                        // packed piece 0 .. 7 (32 values each)
          rr[i] = task & 127;
          p[i] = ld_shared_v4(src + (uint32_t)(rr[i] * 128) + (((uint32_t)cc[i] ^ (uint32_t)(rr[i] & 7)) << 4));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t o[8];
          split16(p[i].x, o[0], o[1]);
          split16(p[i].y, o[2], o[3]);
          split16(p[i].z, o[4], o[5]);
          split16(p[i].w, o[6], o[7]);
          // piece c holds K values 32c .. 32c+31 = int8 bytes 32c .. of the row: K atom c >> 2, 16-byte pieces 2(c & 3), +1
          const uint32_t rowp = dst + (uint32_t)((cc[i] >> 2) * kOAtomBytes + rr[i] * 128), x = (uint32_t)(rr[i] & 7);
          const uint32_t j0 = (uint32_t)(2 * (cc[i] & 3));
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rowp + ((j0 ^ x) << 4)), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rowp + (((j0 + 1) ^ x) << 4)), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
        }
      }
      mbar_arrive_warp(smem_u32(&bars->p_empty[ps]));  // every loaded value has been consumed by the stores above
      fence_proxy_async_smem();  // the tensor core reads the stage through the async proxy
      __syncwarp();
      if (lane == 0) {
        const uint32_t ready = smem_u32(&bars->op_ready[s]);
        if (rank == 0) mbar_arrive(ready); else mbar_arrive_cluster(cluster_map_shared(ready, 0));
      }
    }
  }

  // Nobody leaves while the other CTA may still signal it: the leader's commits to the peer's barriers complete with
  // the MMAs, which both CTAs' epilogues have waited for (accumulator barrier); the peer's arrivals on the leader's
  // barriers were made before this barrier.  The last "operand stage free" commits are awaited by one thread below.
  if (tid == 32 * kAWarp0 && total_steps > 0) {
    for (int back = 0; back < kOStages && back < total_steps; ++back) {
      const int st = total_steps - 1 - back, s = st % kOStages, ph = (st / kOStages) & 1;
      if (!mbar_wait(smem_u32(&bars->op_empty[s]), ph)) { atomicCAS(status, 0u, 0xA60u + s); break; }
    }
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn unpack_encode_fn() {
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

// packed operand [rows, k / 2 bytes] with a row stride of ld_words 32-bit words; boxes of 128 bytes x box_rows rows
int make_map_packed(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld_words, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)(k / 2), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)(ld_words * 4)};
  const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = unpack_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QO_ERR_CUDA, "int4_matmul: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return QO_OK;
}

// CTA pairs of this kernel the device runs at once (0 if the query fails); cached per device
template <typename OutT, bool GATHER>
int max_pairs(int dev) {
  static int cached[64] = {};
  int& c = cached[dev & 63];
  if (c == 0) {
    auto kern = gemm_s4_unpack_kernel<OutT, GATHER>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) { (void)cudaGetLastError(); c = -1; return 0; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int nclusters = 0;
    if (cudaOccupancyMaxActiveClusters(&nclusters, kern, &cfg) != cudaSuccess) { (void)cudaGetLastError(); nclusters = -1; }
    c = nclusters > 0 ? nclusters : -1;
  }
  return c > 0 ? c : 0;
}

template <typename OutT, bool GATHER>
int launch_typed(const int32_t* a, int64_t lda, const int32_t* b, int64_t ldb, const float* sa, const float* sb, void* out,
                 int32_t* acc_out, const void* bias, int64_t t, int64_t k, int64_t n, uint32_t* status, const GatherDsts& dsts,
                 cudaStream_t stream) {
  int dev = 0;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  const int pairs_max = max_pairs<OutT, GATHER>(dev);
  if (pairs_max <= 0) return QO_ERR_UNSUPPORTED;
  CUtensorMap a_map, b_map;
  int rc = make_map_packed(&a_map, a, t, k, lda, kBM);
  if (rc) return rc;
  if ((rc = make_map_packed(&b_map, b, n, k, ldb, kBNh))) return rc;
  const int64_t ntiles = ((t + 2 * kBM - 1) / (2 * kBM)) * ((n + kBN - 1) / kBN);
  const int pairs = (int)(ntiles < pairs_max ? ntiles : pairs_max);
  // tiles of a last wave that would occupy at most half of the pairs are cut into halves of 128 columns
  const int64_t whole = (ntiles / pairs) * pairs, rest = ntiles - whole;
  const bool cut = rest > 0 && 2 * rest <= pairs;
  const int items = (int)(cut ? whole + 2 * rest : ntiles), cut_from = cut ? (int)whole : 0x7fffffff;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  QO_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_s4_unpack_kernel<OutT, GATHER>, a_map, b_map, sa, sb, reinterpret_cast<OutT*>(out), acc_out,
                                 reinterpret_cast<const OutT*>(bias), (int)t, (int)n, (int)k, items, cut_from, status, dsts));
  return check_launch("gemm_s4_unpack_kernel");
}

}  // namespace

// shapes the in-kernel-unpack GEMM takes: both operands with K contiguous and 16-byte aligned rows, K a multiple of
// 256 (a ragged stage would be filled with zero BYTES by TMA, which are not zero CODES in offset binary)
bool gemm_unpack_supported(int64_t t, int64_t k, int64_t n, const void* a, int64_t lda, const void* b, int64_t bsk, int64_t bsn) {
  if (k < kKStage || (k % kKStage) != 0 || k > 131072) return false;
  if (n % 8) return false;  // 16-byte output stores
  if (bsk != 1 || (bsn % 4) != 0 || (lda % 4) != 0) return false;
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(b) % 16) return false;
  if (t > 0x7fffff00LL || n > 0x7fffff00LL) return false;
  return unpack_encode_fn() != nullptr;
}

// Shapes for which the kernel is the better choice: enough 256 x 256 tiles to keep the CTA pairs busy, and a row count
// that 256-row tiles do not pad by much.  Fewer rows run on the single-CTA kernels (which split K over clusters).
bool gemm_unpack_preferred(int64_t t, int64_t k, int64_t n) {
  (void)k;
  if (current_kernel_policy() == 3) return false;
  const int64_t tiles = ((t + 2 * kBM - 1) / (2 * kBM)) * ((n + kBN - 1) / kBN);
  const int64_t rows256 = ((t + 255) / 256) * 256, rows128 = ((t + 127) / 128) * 128;
  return n >= kBN && tiles >= 48 && rows256 * 8 <= rows128 * 9;
}

// returns QO_ERR_UNSUPPORTED without a message when the device cannot co-schedule CTA pairs of this kernel
int launch_gemm_unpack(const int32_t* a, int64_t lda, const int32_t* b, int64_t ldb, const float* sa, const float* sb, void* out,
                       int out_dtype, int64_t t, int64_t k, int64_t n, int32_t* acc_out, const void* bias, uint32_t* status,
                       cudaStream_t stream, const GatherDsts* gather) {
  if (out_dtype != QO_F16 && out_dtype != QO_BF16) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: out_dtype must be QO_F16 or QO_BF16");
  if (bias && reinterpret_cast<uintptr_t>(bias) % 4) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: bias must be 4-byte aligned");
  if (gather != nullptr) {
    if (n % 16) return fail(QO_ERR_UNSUPPORTED, "w4a4_linear_gather: n_out must be a multiple of 16");
    for (int d = 0; d < gather->n_dst; ++d)
      if (!gather->ptr[d] || reinterpret_cast<uintptr_t>(gather->ptr[d]) % 32)
        return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear_gather: destination %d is null or not 32-byte aligned", d);
    if (out_dtype == QO_F16) return launch_typed<__half, true>(a, lda, b, ldb, sa, sb, nullptr, nullptr, bias, t, k, n, status, *gather, stream);
    return launch_typed<__nv_bfloat16, true>(a, lda, b, ldb, sa, sb, nullptr, nullptr, bias, t, k, n, status, *gather, stream);
  }
  if (reinterpret_cast<uintptr_t>(out) % 16 || (acc_out && reinterpret_cast<uintptr_t>(acc_out) % 16))
    return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: outputs of the tcgen05 kernel must be 16-byte aligned");
  const GatherDsts none = {};
  if (out_dtype == QO_F16) return launch_typed<__half, false>(a, lda, b, ldb, sa, sb, out, acc_out, bias, t, k, n, status, none, stream);
  return launch_typed<__nv_bfloat16, false>(a, lda, b, ldb, sa, sb, out, acc_out, bias, t, k, n, status, none, stream);
}

}  // namespace qo
