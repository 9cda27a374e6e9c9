// FlatQuant quantizer, shape-generic SIMT kernel.
//
// Covers every (M, N) and all three activation dtypes; the tcgen05 kernel in flatquant_sm100.cu takes over for
// the 16-bit shapes it supports.  One CTA works on one token at a time (grid-stride over tokens): the token's
// M x N matrix is staged in shared memory in the activation dtype (every value kept there is a value of that dtype:
// X as given, Y and Z after their rounding), the two small products are evaluated with float32 FMA in ascending-k
// order and rounded to the activation dtype where the reference rounds, then the row extremes give the scale and the
// codes are written 8 at a time.  Two buffers of M*N elements: 16-bit inputs up to 51,200 features (28672 = 128 x 224
// and 32768 = 128 x 256 included), float32 inputs up to 25,600.
//
// Numerics follow flatquant_pytorch (reference: src/quant_ops/ops/quantization/flatquant/ops.py:99-117).
#include "qo_internal.cuh"

namespace qo {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerItem = 8;

// MODE 0: int8 codes, 1: packed codes, 2: transform only (float32 Z written to `codes`)
template <typename T, int MODE>
__global__ void __launch_bounds__(kThreads)
flatquant_generic_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ left,
                         const T* __restrict__ right, void* __restrict__ codes, void* __restrict__ scales,
                         int64_t tokens, int m, int n, float clip, int scale_dtype) {
  extern __shared__ __align__(16) unsigned char smem_bytes[];
  const int feat = m * n;
  T* bufx = reinterpret_cast<T*>(smem_bytes);  // X, later Z
  T* bufy = bufx + feat;                       // Y = round(X . R)
  __shared__ float red_min[kThreads / 32], red_max[kThreads / 32];
  __shared__ float s_scale;

  const int tid = threadIdx.x;
  const int row_groups = (m + kRowsPerItem - 1) / kRowsPerItem;
  const int items = row_groups * n;

  for (int64_t tok = blockIdx.x; tok < tokens; tok += gridDim.x) {
    const T* xr = x + tok * ldx;
    for (int i = tid; i < feat; i += kThreads) bufx[i] = xr[i];
    __syncthreads();

    // Y[r][c] = sum_j X[r][j] * R[j][c]
    for (int it = tid; it < items; it += kThreads) {
      const int c = it % n, r0 = (it / n) * kRowsPerItem;
      float acc[kRowsPerItem];
#pragma unroll
      for (int i = 0; i < kRowsPerItem; ++i) acc[i] = 0.f;
      for (int j = 0; j < n; ++j) {
        const float rv = DT<T>::load(right + (int64_t)j * n + c);
#pragma unroll
        for (int i = 0; i < kRowsPerItem; ++i) {
          const int r = min(r0 + i, m - 1);
          acc[i] = fmaf(DT<T>::load(bufx + r * n + j), rv, acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < kRowsPerItem; ++i)
        if (r0 + i < m) DT<T>::store(bufy + (r0 + i) * n + c, acc[i]);
    }
    __syncthreads();

    // Z[r][c] = sum_k L[k][r] * Y[k][c]   (L^T . Y), written over X
    float lmin = 3.4e38f, lmax = -3.4e38f;
    for (int it = tid; it < items; it += kThreads) {
      const int c = it % n, r0 = (it / n) * kRowsPerItem;
      float acc[kRowsPerItem];
#pragma unroll
      for (int i = 0; i < kRowsPerItem; ++i) acc[i] = 0.f;
      for (int k = 0; k < m; ++k) {
        const float yv = DT<T>::load(bufy + k * n + c);
#pragma unroll
        for (int i = 0; i < kRowsPerItem; ++i) {
          const int r = min(r0 + i, m - 1);
          acc[i] = fmaf(DT<T>::load(left + (int64_t)k * m + r), yv, acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < kRowsPerItem; ++i) {
        if (r0 + i < m) {
          const float z = DT<T>::rnd(acc[i]);
          DT<T>::store(bufx + (r0 + i) * n + c, z);
          lmin = fminf(lmin, z);
          lmax = fmaxf(lmax, z);
        }
      }
    }
    if (MODE == 2) {
      __syncthreads();
      float* zout = reinterpret_cast<float*>(codes) + tok * (int64_t)feat;
      for (int i = tid; i < feat; i += kThreads) zout[i] = DT<T>::load(bufx + i);
      __syncthreads();
      continue;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lmin = fminf(lmin, __shfl_xor_sync(0xffffffffu, lmin, o));
      lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
    }
    if ((tid & 31) == 0) {
      red_min[tid >> 5] = lmin;
      red_max[tid >> 5] = lmax;
    }
    __syncthreads();
    if (tid == 0) {
      float a = red_min[0], b = red_max[0];
      for (int w = 1; w < kThreads / 32; ++w) {
        a = fminf(a, red_min[w]);
        b = fmaxf(b, red_max[w]);
      }
      const float s = token_scale<T>(a, b, clip);
      s_scale = s;
      store_scale(scales, tok, s, scale_dtype);
    }
    __syncthreads();
    const float s = s_scale;

    if (MODE == 1) {
      int32_t* out = reinterpret_cast<int32_t*>(codes) + tok * (int64_t)(feat / 8);
      for (int p = tid; p < feat / 8; p += kThreads) {
        uint32_t w = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) w |= (uint32_t)(quantize_one<T>(DT<T>::load(bufx + p * 8 + i), s) + 8) << (4 * i);
        out[p] = (int32_t)w;
      }
    } else {
      int8_t* out = reinterpret_cast<int8_t*>(codes) + tok * (int64_t)feat;
      for (int i = tid; i < feat; i += kThreads) out[i] = (int8_t)quantize_one<T>(DT<T>::load(bufx + i), s);
    }
    __syncthreads();  // bufx is refilled by the next token
  }
}

template <typename T>
int launch_typed(const void* x, int64_t ldx, const void* left, const void* right, void* codes, void* scales,
                 int64_t tokens, int m, int n, float clip, int pack, int scale_dtype, cudaStream_t stream) {
  const size_t smem = (size_t)2 * m * n * sizeof(T);
  if (smem > 200 * 1024) return fail(QO_ERR_UNSUPPORTED, "flatquant: m*n = %d is too large for the generic kernel", m * n);
  int dev = 0, sms = 148;
  QO_CUDA_TRY(cudaGetDevice(&dev));
  sms = sm_count(dev);
  const int per_sm = smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4);
  const int grid = (int)(tokens < (int64_t)sms * per_sm ? tokens : (int64_t)sms * per_sm);
  auto kern = pack == 2 ? flatquant_generic_kernel<T, 2> : (pack ? flatquant_generic_kernel<T, 1> : flatquant_generic_kernel<T, 0>);
  QO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, kThreads, smem, stream>>>(reinterpret_cast<const T*>(x), ldx, reinterpret_cast<const T*>(left),
                                          reinterpret_cast<const T*>(right), codes, scales, tokens, m, n, clip,
                                          scale_dtype);
  return check_launch("flatquant_generic_kernel");
}

}  // namespace

int launch_flatquant_generic(const void* x, int64_t ldx, const void* left, const void* right, void* codes,
                             void* scales, int64_t tokens, int m, int n, float clip, int in_dtype, int pack,
                             int scale_dtype, cudaStream_t stream) {
  switch (in_dtype) {
    case QO_F32:
      return launch_typed<float>(x, ldx, left, right, codes, scales, tokens, m, n, clip, pack, scale_dtype, stream);
    case QO_F16:
      return launch_typed<__half>(x, ldx, left, right, codes, scales, tokens, m, n, clip, pack, scale_dtype, stream);
    case QO_BF16:
      return launch_typed<__nv_bfloat16>(x, ldx, left, right, codes, scales, tokens, m, n, clip, pack, scale_dtype,
                                         stream);
  }
  return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: unknown in_dtype %d", in_dtype);
}

int launch_transform_generic(const void* x, int64_t ldx, const void* left, const void* right, float* z, int64_t tokens,
                             int m, int n, int in_dtype, cudaStream_t stream) {
  return launch_flatquant_generic(x, ldx, left, right, z, z, tokens, m, n, 1.0f, in_dtype, 2, QO_F32, stream);
}

}  // namespace qo
