// Packed-int4 GEMM, shape- and stride-generic SIMT kernel (dp4a).
//
// Fallback for problems the tcgen05 kernel does not take (ragged K, odd strides, tiny shapes).  64x64 output tile
// per CTA, 256 threads, 4x4 outputs per thread, K consumed 64 int4 values at a time.  Nibbles are widened to
// signed bytes once, on the way into shared memory, in k order, so the inner loop is pure dp4a.
//
// Same arithmetic as the reference kernel (src/quant_ops/ops/quantization/int4_matmul/kernels/
// cuda_int4_matmul_kernel.cu:49-118): int32 accumulation, then (float(acc) * scale_a[row]) * scale_b[col].
#include "qo_internal.cuh"

namespace qo {
namespace {

constexpr int kTile = 64;        // output tile edge
constexpr int kWordsPerStep = 8; // packed words of K per step (= 64 int4 values)
constexpr int kLd = 17;          // unpacked words per row in smem (16 + 1 pad)

// 8 offset-binary nibbles -> two words of four signed bytes each, in k order
__device__ __forceinline__ void widen(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t even = w & 0x0F0F0F0Fu, odd = (w >> 4) & 0x0F0F0F0Fu;
  const uint32_t l = __byte_perm(even, odd, 0x5140), h = __byte_perm(even, odd, 0x7362);
  lo = ((l | 0x80808080u) - 0x08080808u) ^ 0x80808080u;  // per byte: v - 8, no borrow across bytes
  hi = ((h | 0x80808080u) - 0x08080808u) ^ 0x80808080u;
}

template <typename OutT>
__device__ __forceinline__ OutT to_out(float v);
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float from_out(__half v) { return __half2float(v); }
__device__ __forceinline__ float from_out(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename OutT>
__global__ void __launch_bounds__(256)
int4_gemm_generic_kernel(const uint32_t* __restrict__ a, int64_t lda, const uint32_t* __restrict__ b, int64_t bsk,
                         int64_t bsn, const float* __restrict__ sa, const float* __restrict__ sb,
                         OutT* __restrict__ out, int32_t* __restrict__ acc_out, const OutT* __restrict__ bias,
                         int64_t t, int64_t kwords, int64_t n) {
  __shared__ uint32_t as[kTile][kLd];
  __shared__ uint32_t bs[kTile][kLd];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t row0 = (int64_t)blockIdx.y * kTile, col0 = (int64_t)blockIdx.x * kTile;
  int acc[4][4] = {};

  for (int64_t kw0 = 0; kw0 < kwords; kw0 += kWordsPerStep) {
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      const int idx = tid + rep * 256;
      {  // A: words of one row are contiguous
        const int r = idx >> 3, kw = idx & 7;
        uint32_t w = 0x88888888u;  // eight zeros
        if (row0 + r < t && kw0 + kw < kwords) w = a[(row0 + r) * lda + kw0 + kw];
        widen(w, as[r][2 * kw], as[r][2 * kw + 1]);
      }
      {  // B: pick the thread order that walks the unit stride
        int c, kw;
        if (bsn == 1) { c = idx & 63; kw = idx >> 6; } else { c = idx >> 3; kw = idx & 7; }
        uint32_t w = 0x88888888u;
        if (col0 + c < n && kw0 + kw < kwords) w = b[(kw0 + kw) * bsk + (col0 + c) * bsn];
        widen(w, bs[c][2 * kw], bs[c][2 * kw + 1]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      int av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = (int)as[ty * 4 + i][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = (int)bs[tx + 16 * j][kk];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = row0 + ty * 4 + i;
    if (r >= t) continue;
    const float s_row = sa[r];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = col0 + tx + 16 * j;
      if (c >= n) continue;
      OutT v = to_out<OutT>(((float)acc[i][j] * s_row) * sb[c]);
      if (bias != nullptr) v = to_out<OutT>(from_out(v) + from_out(bias[c]));
      out[r * n + c] = v;
      if (acc_out != nullptr) acc_out[r * n + c] = acc[i][j];
    }
  }
}

}  // namespace

int launch_gemm_generic(const int32_t* a, int64_t lda, const int32_t* b, int64_t bsk, int64_t bsn, const float* sa,
                        const float* sb, void* out, int out_dtype, int64_t t, int64_t k, int64_t n, int32_t* acc_out,
                        const void* bias, cudaStream_t stream) {
  dim3 grid((unsigned)((n + kTile - 1) / kTile), (unsigned)((t + kTile - 1) / kTile));
  if (grid.y > 65535) return fail(QO_ERR_UNSUPPORTED, "int4_matmul: %lld rows exceed the generic kernel's grid", (long long)t);
  const uint32_t* ua = reinterpret_cast<const uint32_t*>(a);
  const uint32_t* ub = reinterpret_cast<const uint32_t*>(b);
  if (out_dtype == QO_F16) {
    int4_gemm_generic_kernel<__half><<<grid, 256, 0, stream>>>(ua, lda, ub, bsk, bsn, sa, sb,
                                                               reinterpret_cast<__half*>(out), acc_out,
                                                               reinterpret_cast<const __half*>(bias), t, k / 8, n);
  } else if (out_dtype == QO_BF16) {
    int4_gemm_generic_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        ua, lda, ub, bsk, bsn, sa, sb, reinterpret_cast<__nv_bfloat16*>(out), acc_out,
        reinterpret_cast<const __nv_bfloat16*>(bias), t, k / 8, n);
  } else {
    return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: out_dtype must be QO_F16 or QO_BF16");
  }
  return check_launch("int4_gemm_generic_kernel");
}

}  // namespace qo
