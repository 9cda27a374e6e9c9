// int8 x int8 -> int32 GEMM main loop on CTA pairs (tcgen05 cta_group::2), the kernel for prefill-sized products.
//
// Two CTAs of a thread-block cluster, on the two SMs of one TPC, share a 256 x 256 output tile: each CTA stages its own
// 128 rows of A and only HALF of the tile's 256 B rows (output channels); the tensor cores of the two SMs exchange the B
// halves between themselves.  Per 128-byte K step a CTA therefore moves 32 KB of operands through its shared memory
// for 512 tensor-core cycles, where the single-CTA 128 x 256 tile moves 48 KB: shared-memory bandwidth (TMA writes plus
// the tensor core's operand reads) is what held the single-CTA kernel at about half of the tensor pipe's rate.
//
//   warp 0 (each CTA)   TMA: own A block + own B half into own shared memory; both CTAs' bytes are counted on the
//                       LEADER's "full" barrier (the even-ranked CTA), which the leader arms with the pair's total
//   warp 1 (leader)     issues tcgen05.mma.cta_group::2 kind::i8, M = 256, N = 256, four K = 32 slices per stage;
//                       commits go to the "empty" / "accumulator full" barriers of BOTH CTAs (one commit each, the
//                       peer's barrier addressed through mapa; no multicast form is used)
//   warps 2-5 (each)    epilogue of the CTA's own 128 accumulator rows: (float(acc) * scale_a[row]) * scale_b[col],
//                       16-byte stores; two accumulator stages, so it overlaps the next tile's main loop; when done,
//                       each warp arrives on the leader's "accumulator empty" barrier (remotely from the peer)
//
// Operands are the widened int8 copies (A8 row-major, B8 in 256 x 128-byte blocks) described in int4_gemm_sm100.cu.
// Every mbarrier wait is bounded; the cluster barriers at set-up and tear-down are hardware barriers that every thread
// of both CTAs reaches on every path.  Tensor memory is allocated and freed by warp 1 of each CTA (the paired form of
// the allocation is executed once by each CTA of the pair).
#include <mutex>

#include "qo_internal.cuh"
#include "sm100_ptx.cuh"

namespace qo {
namespace {

using namespace ptx;

constexpr int kBM = 128;   // rows per CTA
constexpr int kBN = 256;   // columns of the pair's tile; each CTA stages kBN / 2 of B's rows
constexpr int kBK = 128;   // K bytes per stage
constexpr int kThreads = 192;
constexpr int kStages = 6;
constexpr int kStageBytes = (kBM + kBN / 2) * kBK;          // 32 KB per CTA
constexpr int kOffSb = kStages * kStageBytes;               // 4 warps x 256 floats
constexpr int kOffBar = kOffSb + 4 * kBN * 4;
constexpr int kSmemBytes = kOffBar + 256 + 1024;

struct PairBars {
  uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2];
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

// first 128-byte row of the slice (channels n0 .., K step ks) of the blocked B operand
__device__ __forceinline__ int b_block_row(int n0, int ks, int ksteps) { return ((n0 >> 8) * ksteps + ks) * 256 + (n0 & 255); }

template <typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_s8_pair_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                    const float* __restrict__ sa, const float* __restrict__ sb, OutT* __restrict__ out,
                    int32_t* __restrict__ acc_out, const OutT* __restrict__ bias, int t, int n, int k,
                    uint32_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PairBars* bars = reinterpret_cast<PairBars*>(smem + kOffBar);
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_cta_rank();            // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tiles_n = (n + kBN - 1) / kBN, tiles_m = (t + 2 * kBM - 1) / (2 * kBM);
  const int ntiles = tiles_m * tiles_n, ksteps = (k + kBK - 1) / kBK;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(smem_u32(&bars->full[i]), 1); mbar_init(smem_u32(&bars->empty[i]), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&bars->acc_full[i]), 1); mbar_init(smem_u32(&bars->acc_empty[i]), 8); }
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
    if (lane == 0) {
      int step = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < ntiles; tile += npairs) {
        const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
        for (int ks = 0; ks < ksteps; ++ks, ++step) {
          const int s = step % kStages, ph = (step / kStages) & 1;
          if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1)) { atomicCAS(status, 0u, 0x900u + s); ok = false; break; }
          const uint32_t full_local = smem_u32(&bars->full[s]);
          if (rank == 0) mbar_arrive_expect_tx(full_local, 2 * kStageBytes);  // the pair's bytes land on the leader's barrier
          const uint32_t full_leader = cluster_map_shared(full_local, 0);
          const uint32_t dst = smem_base + s * kStageBytes;
          tma_load_2d_pair(dst, &a_map, full_leader, ks * kBK, mb * 2 * kBM + (int)rank * kBM);
          tma_load_2d_pair(dst + kBM * kBK, &b_map, full_leader, 0, b_block_row(nb * kBN + (int)rank * (kBN / 2), ks, ksteps));
        }
      }
      // every commit aimed at this CTA's "empty" barriers has to land before the CTA may leave: wait for the last use
      // of each stage (a stage that was never filled has nothing pending)
      for (int back = 0; ok && back < kStages && back < step; ++back) {
        const int st = step - 1 - back, s = st % kStages, ph = (st / kStages) & 1;
        if (!mbar_wait(smem_u32(&bars->empty[s]), ph)) { atomicCAS(status, 0u, 0x908u + s); break; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(2, 1, 1, 0, 0, 2 * kBM, kBN);  // s32 accumulators, s8 x s8, both K-major, M = 256 over the pair
      int step = 0, lt = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < ntiles; tile += npairs, ++lt) {
        const int as = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&bars->acc_empty[as]), aph ^ 1)) { atomicCAS(status, 0u, 0x910u + as); break; }
        tc_fence_after();
        for (int ks = 0; ks < ksteps; ++ks, ++step) {
          const int s = step % kStages, ph = (step / kStages) & 1;
          if (!mbar_wait(smem_u32(&bars->full[s]), ph)) { atomicCAS(status, 0u, 0x920u + s); ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_base + s * kStageBytes, b_base = a_base + kBM * kBK;
#pragma unroll
          for (int j = 0; j < kBK / 32; ++j) {
            const uint64_t ad = umma_smem_desc_sw128(a_base + j * 32, 16, 1024);
            const uint64_t bd = umma_smem_desc_sw128(b_base + j * 32, 16, 1024);
            mma_i8_ss_pair(tmem + as * kBN, ad, bd, idesc, (ks | j) != 0);
          }
          const uint32_t e = smem_u32(&bars->empty[s]);
          mma_commit_pair(e);
          mma_commit_pair(cluster_map_shared(e, 1));
        }
        if (ok) {
          const uint32_t f = smem_u32(&bars->acc_full[as]);
          mma_commit_pair(f);
          mma_commit_pair(cluster_map_shared(f, 1));
        }
      }
    }
  } else {
    const int q = warp & 3;
    float* sb_s = reinterpret_cast<float*>(smem + kOffSb) + (warp - 2) * kBN;
    int lt = 0;
    for (int tile = pair; tile < ntiles; tile += npairs, ++lt) {
      const int mb = tile / tiles_n, nb = tile - mb * tiles_n;
      const int as = lt & 1, aph = (lt >> 1) & 1;
      const int row = mb * 2 * kBM + (int)rank * kBM + q * 32 + lane;
      const bool row_ok = row < t;
      const float s_row = row_ok ? sa[row] : 0.f;
      __syncwarp();
      for (int i = lane; i < kBN; i += 32) sb_s[i] = (nb * kBN + i < n) ? sb[nb * kBN + i] : 0.f;
      __syncwarp();
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_full[as]), aph))) { atomicCAS(status, 0u, 0x930u + as); break; }
      tc_fence_after();
#pragma unroll 2
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + as * kBN + c0, v);
        tmem_ld_wait();
        const int col0 = nb * kBN + c0;
        if (!(row_ok && col0 < n)) continue;
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_map_shared(smem_u32(&bars->acc_empty[as]), 0));  // the leader issues the MMAs
    }
  }

  // Nobody leaves while the other CTA may still signal it or read its shared memory: the leader's last commits have
  // landed (the producers waited for them above, the epilogues for the accumulator barriers), the peer's arrivals on the
  // leader's barriers were made before this barrier.
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

EncodeTiledFn pair_encode_fn() {
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

int make_map_rows(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = pair_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QO_ERR_CUDA, "int4_matmul: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return QO_OK;
}

// CTA pairs of this kernel the device runs at once (0 if the query fails); cached per device
template <typename OutT>
int max_pairs(int dev) {
  static int cached[64] = {};
  int& c = cached[dev & 63];
  if (c == 0) {
    auto kern = gemm_s8_pair_kernel<OutT>;
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

template <typename OutT>
int launch_pair_typed(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out, int32_t* acc_out,
                      const void* bias, int64_t t, int64_t k, int64_t n, uint32_t* status, cudaStream_t stream) {
  int dev = 0;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  const int pairs_max = max_pairs<OutT>(dev);
  if (pairs_max <= 0) return QO_ERR_UNSUPPORTED;
  CUtensorMap a_map, b_map;
  int rc = make_map_rows(&a_map, a8, t, k, kBM);
  if (rc) return rc;
  const int64_t b_rows = ((n + 255) / 256) * ((k + kBK - 1) / kBK) * 256;
  if ((rc = make_map_rows(&b_map, b8, b_rows, kBK, kBN / 2))) return rc;
  const int64_t ntiles = ((t + 2 * kBM - 1) / (2 * kBM)) * ((n + kBN - 1) / kBN);
  const int pairs = (int)(ntiles < pairs_max ? ntiles : pairs_max);
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
  QO_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_s8_pair_kernel<OutT>, a_map, b_map, sa, sb, reinterpret_cast<OutT*>(out), acc_out,
                                 reinterpret_cast<const OutT*>(bias), (int)t, (int)n, (int)k, status));
  return check_launch("gemm_s8_pair_kernel");
}

}  // namespace

// The CTA-pair kernel takes products with enough 256 x 256 tiles to keep the pairs busy; returns QO_ERR_UNSUPPORTED
// (without an error message) when it does not take the shape or the device cannot co-schedule CTA pairs.
int launch_gemm_sm100_pair(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out, int out_dtype,
                           int64_t t, int64_t k, int64_t n, int32_t* acc_out, const void* bias, uint32_t* status,
                           cudaStream_t stream) {
  if (pair_encode_fn() == nullptr) return QO_ERR_UNSUPPORTED;
  if (out_dtype == QO_F16) return launch_pair_typed<__half>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream);
  if (out_dtype == QO_BF16) return launch_pair_typed<__nv_bfloat16>(a8, b8, sa, sb, out, acc_out, bias, t, k, n, status, stream);
  return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: out_dtype must be QO_F16 or QO_BF16");
}

}  // namespace qo
