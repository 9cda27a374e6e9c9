// Bandwidth-bound helpers around the two hot kernels: dequantize, pack / unpack, weight quantizer.
// Each thread moves 16 bytes of codes at a time; grids are sized from the element count.
#include "qo_internal.cuh"

namespace qo {
namespace {

constexpr int kThreads = 256;

// ---- dequantize: reference src/quant_ops/ops/quantization/flatquant/ops.py:156-178 ----------------
// packed: one thread per half word -> 4 floats, so that consecutive lanes write consecutive 16-byte pieces (a warp's
// store covers 512 contiguous bytes); four items per thread are in flight.  The output is 8x the input: the kernel is
// bound by HBM writes.
// A block works on whole rows (tokens), so the row's scale is read once and no piece needs a division to find its row.
__global__ void __launch_bounds__(kThreads)
dequant_packed_kernel(const uint32_t* __restrict__ words, const void* __restrict__ scales, float* __restrict__ out,
                      int64_t tokens, int words_per_row, int scale_dtype) {
  constexpr int kUnroll = 4;
  const int pieces = words_per_row * 2;  // 16-byte output pieces per row
  for (int64_t row = blockIdx.x; row < tokens; row += gridDim.x) {
    const float s = load_scale(scales, row, scale_dtype);
    const uint32_t* wrow = words + row * words_per_row;
    float4* orow = reinterpret_cast<float4*>(out) + row * pieces;
    for (int p0 = threadIdx.x; p0 < pieces; p0 += kThreads * kUnroll) {
      uint32_t w[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int p = p0 + u * kThreads;
        if (p < pieces) w[u] = wrow[p >> 1] >> (16 * (p & 1));  // the four nibbles of this half word
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int p = p0 + u * kThreads;
        if (p < pieces) {
          float4 o;
          o.x = (float)((int)(w[u] & 0xF) - 8) * s;
          o.y = (float)((int)((w[u] >> 4) & 0xF) - 8) * s;
          o.z = (float)((int)((w[u] >> 8) & 0xF) - 8) * s;
          o.w = (float)((int)((w[u] >> 12) & 0xF) - 8) * s;
          __stcs(orow + p, o);  // streaming store: the output is not read back by this kernel
        }
      }
    }
  }
}

// int8 codes: one thread per element group of 4 when aligned, scalar otherwise
__global__ void __launch_bounds__(kThreads)
dequant_int8_kernel(const int8_t* __restrict__ codes, const void* __restrict__ scales, float* __restrict__ out,
                    int64_t tokens, int64_t features, int scale_dtype) {
  const int64_t total = tokens * features;
  if ((features & 3) == 0) {
    // a block works on whole rows: the scale is read once per row, no group needs a division to find its row
    constexpr int kUnroll = 4;
    const int groups = (int)(features >> 2);  // groups of 4 codes per row
    for (int64_t row = blockIdx.x; row < tokens; row += gridDim.x) {
      const float s = load_scale(scales, row, scale_dtype);
      const char4* crow = reinterpret_cast<const char4*>(codes + row * features);
      float4* orow = reinterpret_cast<float4*>(out + row * features);
      for (int g0 = threadIdx.x; g0 < groups; g0 += kThreads * kUnroll) {
        char4 c[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (g0 + u * kThreads < groups) c[u] = crow[g0 + u * kThreads];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (g0 + u * kThreads < groups)
            __stcs(orow + g0 + u * kThreads, make_float4((float)c[u].x * s, (float)c[u].y * s, (float)c[u].z * s, (float)c[u].w * s));
      }
    }
  } else {
    for (int64_t i = blockIdx.x * (int64_t)kThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kThreads)
      out[i] = (float)codes[i] * load_scale(scales, i / features, scale_dtype);
  }
}

// ---- pack / unpack: reference src/quant_ops/ops/quantization/int4_matmul/ops.py:23-66 --------------
__global__ void __launch_bounds__(kThreads)
pack_kernel(const int8_t* __restrict__ codes, uint32_t* __restrict__ packed, int64_t total_words) {
  for (int64_t i = blockIdx.x * (int64_t)kThreads + threadIdx.x; i < total_words; i += (int64_t)gridDim.x * kThreads) {
    const int2 v = reinterpret_cast<const int2*>(codes)[i];  // 8 codes
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      w |= (uint32_t)((((int)(int8_t)(v.x >> (8 * j))) + 8) & 0xF) << (4 * j);
      w |= (uint32_t)((((int)(int8_t)(v.y >> (8 * j))) + 8) & 0xF) << (4 * (j + 4));
    }
    packed[i] = w;
  }
}

__global__ void __launch_bounds__(kThreads)
unpack_kernel(const uint32_t* __restrict__ packed, int8_t* __restrict__ codes, int64_t total_words) {
  for (int64_t i = blockIdx.x * (int64_t)kThreads + threadIdx.x; i < total_words; i += (int64_t)gridDim.x * kThreads) {
    const uint32_t w = packed[i];
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= (uint32_t)(uint8_t)(int8_t)((int)((w >> (4 * j)) & 0xF) - 8) << (8 * j);
      hi |= (uint32_t)(uint8_t)(int8_t)((int)((w >> (4 * (j + 4))) & 0xF) - 8) << (8 * j);
    }
    reinterpret_cast<int2*>(codes)[i] = make_int2((int)lo, (int)hi);
  }
}

// ---- weight quantizer: one warp per output channel ------------------------------------------------
__global__ void __launch_bounds__(kThreads)
quantize_weights_kernel(const float* __restrict__ w, uint32_t* __restrict__ packed, float* __restrict__ scale,
                        int64_t rows, int64_t k) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t r = blockIdx.x * (int64_t)(kThreads / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
    const float* wr = w + r * k;
    float am = 0.f;
    for (int64_t i = lane; i < k; i += 32) am = fmaxf(am, fabsf(wr[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float s = fmaxf(__fdiv_rn(am, 7.0f), 1e-8f);
    if (lane == 0) scale[r] = s;
    for (int64_t p = lane; p < k / 8; p += 32) {
      uint32_t word = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float q = fminf(fmaxf(rintf(__fdiv_rn(wr[p * 8 + i], s)), -8.f), 7.f);
        word |= (uint32_t)((int)q + 8) << (4 * i);
      }
      packed[r * (k / 8) + p] = word;
    }
  }
}

inline int grid_for(int64_t work_items) {
  int64_t blocks = (work_items + kThreads - 1) / kThreads;
  const int64_t cap = 148LL * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

int launch_dequantize(const void* codes, const void* scales, float* out, int64_t tokens, int64_t features, int packed,
                      int scale_dtype, cudaStream_t stream) {
  if (packed) {
    const int64_t wpr = features / 8;
    const int64_t cap = 148LL * 8 * 8;  // rows in flight: eight blocks per SM, a few rounds
    dequant_packed_kernel<<<(int)(tokens < cap ? tokens : cap), kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(codes), scales, out, tokens,
                                                                                     (int)wpr, scale_dtype);
    return check_launch("dequant_packed_kernel");
  }
  dequant_int8_kernel<<<grid_for(tokens * features / 16 + 1), kThreads, 0, stream>>>(
      reinterpret_cast<const int8_t*>(codes), scales, out, tokens, features, scale_dtype);
  return check_launch("dequant_int8_kernel");
}

int launch_pack(const int8_t* codes, int32_t* packed, int64_t rows, int64_t features, cudaStream_t stream) {
  const int64_t words = rows * (features / 8);
  pack_kernel<<<grid_for(words), kThreads, 0, stream>>>(codes, reinterpret_cast<uint32_t*>(packed), words);
  return check_launch("pack_kernel");
}

int launch_unpack(const int32_t* packed, int8_t* codes, int64_t rows, int64_t features, cudaStream_t stream) {
  const int64_t words = rows * (features / 8);
  unpack_kernel<<<grid_for(words), kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(packed), codes, words);
  return check_launch("unpack_kernel");
}

int launch_quantize_weights(const float* w, int32_t* packed, float* scale, int64_t rows, int64_t k,
                            cudaStream_t stream) {
  quantize_weights_kernel<<<grid_for(rows * 32), kThreads, 0, stream>>>(w, reinterpret_cast<uint32_t*>(packed), scale,
                                                                        rows, k);
  return check_launch("quantize_weights_kernel");
}

}  // namespace qo
