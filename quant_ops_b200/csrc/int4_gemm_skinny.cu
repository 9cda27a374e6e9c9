// Packed-int4 GEMM for a handful of activation rows (decode steps: 1 .. 32 tokens), a weight-streaming kernel.
//
// With so few rows the product is bound by reading the packed weights once from HBM (Nout * K / 2 bytes); a
// 128-row tcgen05 tile would spend at least three quarters of its rows on padding and would need the weights widened
// to int8 in memory first, which doubles the bytes.  Here the weights stay packed all the way into registers:
//
//   * one CTA owns 16 or 32 output channels (rows of the [Nout, K/8] weight matrix); per 16 channels, 8 warps split
//     K into 8 contiguous slices and add their partial sums through shared memory at the end;
//   * a lane loads 16 bytes of a weight row at a time (four lanes cover 64 contiguous bytes of one row, a warp 16
//     rows, consecutive loads of a warp walk along the rows), four chunks of 128 values per batch, and the next
//     batch is requested before the current one is multiplied;
//   * the activation rows (K / 2 bytes per token) are copied into shared memory once per CTA with cp.async while the
//     first weight loads are in flight (rows padded by 64 bytes so that the fragment reads are conflict-free); with
//     more tokens than fit, two row tiles share one copy (32 channels per CTA), and beyond that the rows are read
//     through L1 / L2 instead;
//   * nibbles become int8 operands without sign extension: x ^ 0x88888888 turns the offset-binary nibbles into
//     two's-complement nibbles, and a nibble placed in the HIGH half of a byte is the int8 value 16 * n.  The even
//     and the odd elements of a word make one operand register each; activations are treated identically, so both
//     sides agree on the (permuted) order of K, and every product carries the factor 256, removed exactly by an
//     arithmetic shift at the end (|256 * acc| < 2^31 for K <= 131072);
//   * the products run on mma.sync m16n8k32 (int8): channels are the 16 rows, 8 tokens the columns.
//
// Arithmetic as in the reference kernel (src/quant_ops/ops/quantization/int4_matmul/kernels/
// cuda_int4_matmul_kernel.cu:49-118): int32 accumulation, then (float(acc) * scale_a[row]) * scale_b[col].
#include "qo_internal.cuh"
#include "sm100_ptx.cuh"

namespace qo {
namespace {

constexpr int kSlices = 8;       // warps per 16 output channels: each takes a contiguous eighth of K
constexpr int kChunkWords = 16;  // packed words of one weight row per chunk (4 lanes x 16 bytes)
constexpr int kBatch = 4;        // chunks per batch of weight loads (two batches in flight)
constexpr size_t kSmemOptIn = 227 * 1024;  // shared memory one CTA may use on sm_100 (static + dynamic)
// bytes of the partial-sum exchange, a static array of the kernel below
constexpr size_t red_bytes(int nt, int rt) { return (size_t)kSlices * rt * nt * 16 * 9 * sizeof(int); }

template <typename OutT>
__device__ __forceinline__ OutT to_out(float v);
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float from_out(__half v) { return __half2float(v); }
__device__ __forceinline__ float from_out(__nv_bfloat16 v) { return __bfloat162float(v); }

// packed word -> (even elements, odd elements) as int8 bytes holding 16 * value
__device__ __forceinline__ void split16(uint32_t w, uint32_t& even, uint32_t& odd) {
  const uint32_t t = w ^ 0x88888888u;
  even = (t << 4) & 0xF0F0F0F0u;
  odd = t & 0xF0F0F0F0u;
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const uint32_t* p) {  // weights are read once: do not keep them in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// NT = number of 8-token column tiles (tokens <= 8 * NT); RT = row tiles of 16 channels per CTA;
// STAGED = activation rows are copied to shared memory (row stride nchunks * 64 + 64 bytes)
template <int NT, int RT, bool STAGED, typename OutT>
__global__ void __launch_bounds__(kSlices * RT * 32, RT == 1 ? 2 : 1)
int4_gemm_skinny_kernel(const uint32_t* __restrict__ a, int64_t lda, const uint32_t* __restrict__ b, int64_t ldb,
                        const float* __restrict__ sa, const float* __restrict__ sb, OutT* __restrict__ out,
                        int32_t* __restrict__ acc_out, const OutT* __restrict__ bias, int tokens, int nchunks, int64_t n,
                        int weights_first) {
  constexpr int kThreads = kSlices * RT * 32;
  __shared__ int red[kSlices * RT][NT][16][8 + 1];
  extern __shared__ uint4 act[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int rt = warp % RT, slice = warp / RT;
  const int64_t n0 = ((int64_t)blockIdx.x * RT + rt) * 16;
  const uint4 zero4 = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);  // eight zeros per word
  const int stride4 = nchunks * 4 + 4;  // activation row stride in shared memory, in 16-byte units

  // Launched with programmatic stream serialization, the kernel may start while its predecessor in the stream (the
  // activation quantizer) still runs.  weights_first: the weights are known not to come from that predecessor, so the
  // first batch of weight loads is issued before the wait and overlaps it; everything else comes after the wait.
  if (!weights_first) ptx::grid_dependency_wait();
  auto stage_activations = [&]() {
    if (STAGED) {
      const int per_row = nchunks * 4, total = tokens * per_row;
      const uint32_t base = (uint32_t)__cvta_generic_to_shared(act);
      for (int p = threadIdx.x; p < total; p += kThreads) {
        const int tok = p / per_row, q = p - tok * per_row;
        cp_async16(base + (uint32_t)(tok * stride4 + q) * 16u, a + (int64_t)tok * lda + (int64_t)q * 4);
      }
    }
  };
  if (!weights_first) stage_activations();

  const int per = (nchunks + kSlices - 1) / kSlices;
  const int cb = slice * per, ce = min(nchunks, cb + per);
  const bool row0_ok = n0 + g < n, row1_ok = n0 + g + 8 < n;
  const uint32_t* w0p = b + (n0 + g) * ldb + 4 * t4;
  const uint32_t* w1p = b + (n0 + g + 8) * ldb + 4 * t4;
  bool tok_ok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) tok_ok[nt] = nt * 8 + g < tokens;

  int acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0;

  uint4 w0[2][kBatch], w1[2][kBatch];
  auto load = [&](int buf, int c0) {
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int c = c0 + u;
      w0[buf][u] = (c < ce && row0_ok) ? ld_stream(w0p + (int64_t)c * kChunkWords) : zero4;
      w1[buf][u] = (c < ce && row1_ok) ? ld_stream(w1p + (int64_t)c * kChunkWords) : zero4;
    }
  };
  auto compute = [&](int buf, int c0) {
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int c = c0 + u;
      if (c >= ce) break;
      uint4 x[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (!tok_ok[nt]) x[nt] = zero4;
        else if (STAGED) x[nt] = act[(nt * 8 + g) * stride4 + c * 4 + t4];
        else x[nt] = __ldg(reinterpret_cast<const uint4*>(a + (int64_t)(nt * 8 + g) * lda + (int64_t)c * kChunkWords + 4 * t4));
      }
      const uint32_t w0w[4] = {w0[buf][u].x, w0[buf][u].y, w0[buf][u].z, w0[buf][u].w};
      const uint32_t w1w[4] = {w1[buf][u].x, w1[buf][u].y, w1[buf][u].z, w1[buf][u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a0, a1, a2, a3;
        split16(w0w[j], a0, a2);  // row g:     slots t4 (even elements) and 4 + t4 (odd elements)
        split16(w1w[j], a1, a3);  // row g + 8
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t xw = j == 0 ? x[nt].x : (j == 1 ? x[nt].y : (j == 2 ? x[nt].z : x[nt].w));
          uint32_t b0, b1;
          split16(xw, b0, b1);
          mma_s8(acc[nt], a0, a1, a2, a3, b0, b1);
        }
      }
    }
  };

  load(0, cb);
  if (weights_first) {
    ptx::grid_dependency_wait();
    stage_activations();
  }
  if (STAGED) {
    cp_async_wait_all();
    __syncthreads();
  }
  for (int c0 = cb; c0 < ce; c0 += 2 * kBatch) {
    load(1, c0 + kBatch);
    compute(0, c0);
    load(0, c0 + 2 * kBatch);
    compute(1, c0 + kBatch);
  }

  // fragment: c0 (row g, col 2 t4), c1 (row g, col 2 t4 + 1), c2 / c3 the same for row g + 8
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    red[warp][nt][g][2 * t4] = acc[nt][0];
    red[warp][nt][g][2 * t4 + 1] = acc[nt][1];
    red[warp][nt][g + 8][2 * t4] = acc[nt][2];
    red[warp][nt][g + 8][2 * t4 + 1] = acc[nt][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < RT * NT * 128; idx += kThreads) {
    const int r = idx & 15, col = (idx >> 4) & 7, nt = (idx >> 7) % NT, tile = idx / (NT * 128);
    const int tok = nt * 8 + col;
    const int64_t ch = ((int64_t)blockIdx.x * RT + tile) * 16 + r;
    if (tok >= tokens || ch >= n) continue;
    int sum = 0;
#pragma unroll
    for (int w = 0; w < kSlices; ++w) sum += red[w * RT + tile][nt][r][col];
    sum >>= 8;  // both operands carried the factor 16
    OutT v = to_out<OutT>(((float)sum * sa[tok]) * sb[ch]);
    if (bias != nullptr) v = to_out<OutT>(from_out(v) + from_out(bias[ch]));
    out[(int64_t)tok * n + ch] = v;
    if (acc_out != nullptr) acc_out[(int64_t)tok * n + ch] = sum;
  }
}

// ---- decode steps inside the fused layer: the CTA's weight rows are made RESIDENT in shared memory --------------------
// Inside the fused layer the kernel before this one is the call's own activation quantizer (one CTA per two tokens, a
// chain of latencies of about 6 us), and this kernel may start beside it (programmatic stream serialization).  The
// streaming kernel above can only fetch its first batch of weights before it has to wait for the codes; here every CTA
// (one per SM) copies ALL of its weight rows -- n_out / #SMs channels, e.g. 28 rows of 7 KB = 200 KB for 14336 -> 4096 --
// into shared memory with bulk copies while the quantizer runs, and after the dependency wait only the codes (a few KB
// per token, from L2) are fetched and multiplied.  The weight bytes, the bound of a decode step, move entirely under
// the quantizer.  Rows are padded by 64 bytes so that the fragment reads are conflict-free; the partial sums of the 16
// warps (each takes a sixteenth of K) are added through the same shared memory once the weights are no longer needed.
constexpr int kResWarps = 16;

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// NT = 8-token column tiles, TILES = 16-channel row tiles per CTA (TILES * NT <= 8 keeps the accumulators in registers)
template <int NT, int TILES, typename OutT>
__global__ void __launch_bounds__(kResWarps * 32, 1)
int4_gemm_resident_kernel(const uint32_t* __restrict__ a, int64_t lda, const uint32_t* __restrict__ b, int64_t ldb,
                          const float* __restrict__ sa, const float* __restrict__ sb, OutT* __restrict__ out,
                          int32_t* __restrict__ acc_out, const OutT* __restrict__ bias, int tokens, int nchunks, int64_t n,
                          int cpc, uint32_t* __restrict__ status) {
  extern __shared__ uint4 wsm[];  // weight rows, row stride nchunks * 4 + 4 uint4; later the partial sums
  __shared__ uint64_t bar;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int64_t c0 = (int64_t)blockIdx.x * cpc;
  const int nch = (int)min((int64_t)cpc, n - c0);  // the grid is sized so that every CTA has at least one channel
  const int stride4 = nchunks * 4 + 4;
  const uint32_t bar_a = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar_a, 1);
    ptx::fence_barrier_init();
  }
  __syncthreads();
  // the weights are not written by the kernel before this one (the caller says so): fetch them before the wait
  if (threadIdx.x == 0) {
    const uint32_t row_bytes = (uint32_t)nchunks * 64u;
    ptx::mbar_arrive_expect_tx(bar_a, (uint32_t)nch * row_bytes);
    const uint32_t base = ptx::smem_u32(wsm);
    for (int r = 0; r < nch; ++r) bulk_copy_g2s(base + (uint32_t)(r * stride4) * 16u, b + (c0 + r) * ldb, row_bytes, bar_a);
  }
  ptx::grid_dependency_wait();  // the codes and their scales are complete now

  const uint4 zero4 = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);  // eight zeros per word
  const int per = (nchunks + kResWarps - 1) / kResWarps;
  const int cb = warp * per, ce = min(nchunks, cb + per);
  bool tok_ok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) tok_ok[nt] = nt * 8 + g < tokens;
  auto load_x = [&](uint4 (&x)[NT], int c) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      x[nt] = (tok_ok[nt] && c < ce) ? __ldg(reinterpret_cast<const uint4*>(a + (int64_t)(nt * 8 + g) * lda + (int64_t)c * kChunkWords + 4 * t4)) : zero4;
  };
  uint4 xa[NT], xb[NT];
  load_x(xa, cb);  // the first codes are requested while the last weight rows may still be arriving

  const bool landed = ptx::mbar_wait(bar_a, 0);
  if (!__syncthreads_and(landed)) {  // one decision for the whole CTA
    if (threadIdx.x == 0) atomicCAS(status, 0u, 0xB00u);
    return;  // the outputs stay unwritten; qo_device_status reports the timeout
  }

  int acc[TILES][NT][4];
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[tl][nt][i] = 0;

  auto compute = [&](const uint4 (&x)[NT], int c) {
    if (c >= ce) return;
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl) {
      const int r0 = tl * 16 + g, r1 = r0 + 8;
      if (tl * 16 >= nch) break;  // uniform: this tile has no channel
      const uint4 w0 = r0 < nch ? wsm[r0 * stride4 + c * 4 + t4] : zero4;
      const uint4 w1 = r1 < nch ? wsm[r1 * stride4 + c * 4 + t4] : zero4;
      const uint32_t w0w[4] = {w0.x, w0.y, w0.z, w0.w}, w1w[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a0, a1, a2, a3;
        split16(w0w[j], a0, a2);
        split16(w1w[j], a1, a3);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t xw = j == 0 ? x[nt].x : (j == 1 ? x[nt].y : (j == 2 ? x[nt].z : x[nt].w));
          uint32_t b0, b1;
          split16(xw, b0, b1);
          mma_s8(acc[tl][nt], a0, a1, a2, a3, b0, b1);
        }
      }
    }
  };
  for (int c = cb; c < ce; c += 2) {
    load_x(xb, c + 1);
    compute(xa, c);
    load_x(xa, c + 2);
    compute(xb, c + 1);
  }

  // partial sums of the 16 warps through the shared memory that held the weights
  __syncthreads();
  int* red = reinterpret_cast<int*>(wsm);  // [warp][tile][nt][16][9]
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      int* p = red + (((warp * TILES + tl) * NT + nt) * 16) * 9;
      p[g * 9 + 2 * t4] = acc[tl][nt][0];
      p[g * 9 + 2 * t4 + 1] = acc[tl][nt][1];
      p[(g + 8) * 9 + 2 * t4] = acc[tl][nt][2];
      p[(g + 8) * 9 + 2 * t4 + 1] = acc[tl][nt][3];
    }
  __syncthreads();
  for (int idx = threadIdx.x; idx < TILES * NT * 128; idx += kResWarps * 32) {
    const int r = idx & 15, col = (idx >> 4) & 7, nt = (idx >> 7) % NT, tl = idx / (NT * 128);
    const int tok = nt * 8 + col, chl = tl * 16 + r;
    if (tok >= tokens || chl >= nch) continue;
    int sum = 0;
#pragma unroll
    for (int w = 0; w < kResWarps; ++w) sum += red[(((w * TILES + tl) * NT + nt) * 16 + r) * 9 + col];
    sum >>= 8;  // both operands carried the factor 16
    const int64_t ch = c0 + chl;
    OutT v = to_out<OutT>(((float)sum * sa[tok]) * sb[ch]);
    if (bias != nullptr) v = to_out<OutT>(from_out(v) + from_out(bias[ch]));
    out[(int64_t)tok * n + ch] = v;
    if (acc_out != nullptr) acc_out[(int64_t)tok * n + ch] = sum;
  }
}

// the resident-weights kernel for this problem, or QO_ERR_UNSUPPORTED (no message) when its limits do not hold
template <int NT, int TILES, typename OutT>
int launch_resident_cfg(const uint32_t* a, int64_t lda, const uint32_t* b, int64_t ldb, const float* sa, const float* sb, void* out,
                        int32_t* acc_out, const void* bias, int tokens, int nchunks, int64_t n, int cpc, int grid, size_t smem,
                        uint32_t* status, cudaStream_t stream) {
  auto kern = int4_gemm_resident_kernel<NT, TILES, OutT>;
  int dev = 0;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    QO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kSmemOptIn - 64)));
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kResWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  QO_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a, lda, b, ldb, sa, sb, reinterpret_cast<OutT*>(out), acc_out,
                                 reinterpret_cast<const OutT*>(bias), tokens, nchunks, n, cpc, status));
  return check_launch("int4_gemm_resident_kernel");
}

template <typename OutT>
int launch_resident(const uint32_t* a, int64_t lda, const uint32_t* b, int64_t ldb, const float* sa, const float* sb, void* out,
                    int32_t* acc_out, const void* bias, int tokens, int nchunks, int64_t n, cudaStream_t stream) {
  int dev = 0;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  // The kernel before this one (the activation quantizer) holds one SM per token (or two tokens) for its whole run, and a
  // CTA of this kernel, which wants an SM's whole shared memory, could only start there once it has left.  The grid
  // is therefore sized for the SMs that are free NOW: every CTA starts, and fetches its weights, beside the quantizer.
  // (When the rows of so few CTAs would not fit in shared memory, all SMs are used and some CTAs start late.)
  const size_t row = (size_t)nchunks * 64 + 64;
  int sms = max(sm_count(dev) - tokens, sm_count(dev) / 2);
  if ((size_t)((n + sms - 1) / sms) * row > kSmemOptIn - 64) sms = sm_count(dev);
  const int cpc = (int)((n + sms - 1) / sms);           // channels per CTA
  const int grid = (int)((n + cpc - 1) / cpc);
  const int tiles = (cpc + 15) / 16, nt = tokens <= 8 ? 1 : (tokens <= 16 ? 2 : 4);
  size_t smem = (size_t)cpc * row;
  const size_t red = (size_t)kResWarps * tiles * nt * 16 * 9 * sizeof(int);  // the reduction reuses the weight area
  if (red > smem) smem = red;
  if (smem > kSmemOptIn - 64 || tiles * nt > 8 || n < sms) return QO_ERR_UNSUPPORTED;
  uint32_t* status = device_status_word(dev);
  if (!status) return QO_ERR_UNSUPPORTED;
#define QO_RES(NTV, TLV) return launch_resident_cfg<NTV, TLV, OutT>(a, lda, b, ldb, sa, sb, out, acc_out, bias, tokens, nchunks, n, cpc, grid, smem, status, stream)
  if (nt == 1) {
    if (tiles <= 1) QO_RES(1, 1);
    if (tiles <= 2) QO_RES(1, 2);
    if (tiles <= 4) QO_RES(1, 4);
    QO_RES(1, 8);
  }
  if (nt == 2) {
    if (tiles <= 1) QO_RES(2, 1);
    if (tiles <= 2) QO_RES(2, 2);
    QO_RES(2, 4);
  }
  if (tiles <= 1) QO_RES(4, 1);
  QO_RES(4, 2);
#undef QO_RES
}

template <int NT, int RT, bool STAGED, typename OutT>
int launch_cfg(const uint32_t* a, int64_t lda, const uint32_t* b, int64_t ldb, const float* sa, const float* sb, void* out,
               int32_t* acc_out, const void* bias, int tokens, int nchunks, int64_t n, size_t smem, int weights_first,
               cudaStream_t stream) {
  auto kern = int4_gemm_skinny_kernel<NT, RT, STAGED, OutT>;
  if (smem > 0) {
    int dev = 0;
    QO_CUDA_TRY(cudaGetDevice(&dev));
    static bool configured[64] = {};
    if (!configured[dev & 63]) {
      // static and dynamic shared memory together must stay within the opt-in limit
      QO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kSmemOptIn - red_bytes(NT, RT))));
      configured[dev & 63] = true;
    }
  }
  const unsigned grid = (unsigned)((n + 16 * RT - 1) / (16 * RT));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kSlices * RT * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  QO_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a, lda, b, ldb, sa, sb, reinterpret_cast<OutT*>(out), acc_out,
                                 reinterpret_cast<const OutT*>(bias), tokens, nchunks, n, weights_first));
  return check_launch("int4_gemm_skinny_kernel");
}

template <int NT, typename OutT>
int launch_nt(const uint32_t* a, int64_t lda, const uint32_t* b, int64_t ldb, const float* sa, const float* sb, void* out,
              int32_t* acc_out, const void* bias, int tokens, int nchunks, int64_t n, int weights_first, cudaStream_t stream) {
  const size_t stage = (size_t)tokens * ((size_t)nchunks * 64 + 64);
  if (stage <= 92 * 1024)  // two CTAs of 16 channels per SM
    return launch_cfg<NT, 1, true, OutT>(a, lda, b, ldb, sa, sb, out, acc_out, bias, tokens, nchunks, n, stage, weights_first, stream);
  if (stage + red_bytes(NT, 2) <= kSmemOptIn)  // one CTA of 32 channels per SM shares the copy
    return launch_cfg<NT, 2, true, OutT>(a, lda, b, ldb, sa, sb, out, acc_out, bias, tokens, nchunks, n, stage, weights_first, stream);
  return launch_cfg<NT, 1, false, OutT>(a, lda, b, ldb, sa, sb, out, acc_out, bias, tokens, nchunks, n, 0, weights_first, stream);
}

template <typename OutT>
int launch_t(const uint32_t* a, int64_t lda, const uint32_t* b, int64_t ldb, const float* sa, const float* sb, void* out,
             int32_t* acc_out, const void* bias, int tokens, int nchunks, int64_t n, int weights_first, cudaStream_t stream) {
  if (tokens <= 8) return launch_nt<1, OutT>(a, lda, b, ldb, sa, sb, out, acc_out, bias, tokens, nchunks, n, weights_first, stream);
  if (tokens <= 16) return launch_nt<2, OutT>(a, lda, b, ldb, sa, sb, out, acc_out, bias, tokens, nchunks, n, weights_first, stream);
  return launch_nt<4, OutT>(a, lda, b, ldb, sa, sb, out, acc_out, bias, tokens, nchunks, n, weights_first, stream);
}

}  // namespace

// few rows, weights contiguous along K, K a multiple of 128, rows of both operands 16-byte aligned
bool gemm_skinny_supported(int64_t t, int64_t k, int64_t n, const void* a, int64_t lda, const void* b, int64_t bsk, int64_t bsn) {
  return t >= 1 && t <= 32 && n >= 1 && k >= 128 && k <= 131072 && (k % 128) == 0 && bsk == 1 && (bsn % 4) == 0 && (lda % 4) == 0 &&
         (reinterpret_cast<uintptr_t>(a) % 16) == 0 && (reinterpret_cast<uintptr_t>(b) % 16) == 0 && n <= (int64_t)16 * 0x7fffffff;
}

int launch_gemm_skinny(const int32_t* a, int64_t lda, const int32_t* b, int64_t bsn, const float* sa, const float* sb, void* out,
                       int out_dtype, int64_t t, int64_t k, int64_t n, int32_t* acc_out, const void* bias, cudaStream_t stream,
                       bool weights_first) {
  const uint32_t* ua = reinterpret_cast<const uint32_t*>(a);
  const uint32_t* ub = reinterpret_cast<const uint32_t*>(b);
  const int nchunks = (int)(k / 128);
  if (weights_first) {
    // inside the fused layer: the weights can be fetched in full beside the quantizer that precedes this kernel
    int rc = QO_ERR_UNSUPPORTED;
    if (out_dtype == QO_F16) rc = launch_resident<__half>(ua, lda, ub, bsn, sa, sb, out, acc_out, bias, (int)t, nchunks, n, stream);
    else if (out_dtype == QO_BF16) rc = launch_resident<__nv_bfloat16>(ua, lda, ub, bsn, sa, sb, out, acc_out, bias, (int)t, nchunks, n, stream);
    if (rc != QO_ERR_UNSUPPORTED) return rc;
  }
  if (out_dtype == QO_F16) return launch_t<__half>(ua, lda, ub, bsn, sa, sb, out, acc_out, bias, (int)t, nchunks, n, weights_first ? 1 : 0, stream);
  if (out_dtype == QO_BF16) return launch_t<__nv_bfloat16>(ua, lda, ub, bsn, sa, sb, out, acc_out, bias, (int)t, nchunks, n, weights_first ? 1 : 0, stream);
  return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: out_dtype must be QO_F16 or QO_BF16");
}

}  // namespace qo
