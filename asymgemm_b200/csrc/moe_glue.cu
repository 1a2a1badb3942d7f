// Memory-bound helper kernels around the two grouped GEMMs of an expert-parallel FP8 MoE layer: 1x128 FP8 row
// quantisation, SiLU(gate)*up fused with that quantisation, row gather/scatter between token order and the padded
// contiguous layout, and the router-weighted top-k combine. Callers of the reference do these steps with separate torch
// kernels (asym_gemm/unified_moe/runtime.py:1422-1476,1570,1620-1627; asym_gemm/training/frozen_linear.py:595-693);
// each is one pass over its data here.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/asymgemm_b200.h"

int agb_fail(int code, const char* message);

namespace agb {

constexpr float kFp8Max = 448.0f;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint32_t quantise4(const float (&v)[4], float inv) {
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    out |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  return out;
}

// One warp per (row, 128-column block): scale = max(amax, 1e-4) / 448, q = e4m3(x * (1 / scale)).
// MODE 0: x is bf16 [rows, cols]. MODE 1: x is bf16 [rows, 2*cols] holding gate | up; the value quantised is
// bf16(silu(gate) * up), the activation the reference's CPU MoE bucket forms (csrc/cpu/module.cpp:337-347).
// Smallest power of two >= x (x > 0, finite): what ceil_to_ue8m0 of the quantisers computes (asym_gemm/utils/math.py:17-21).
__device__ __forceinline__ float ceil_pow2(float x) {
  const uint32_t bits = __float_as_uint(x);
  return __uint_as_float((bits & 0x7F800000u) + ((bits & 0x007FFFFFu) ? 0x00800000u : 0u));
}

// `pow2_scales`: round every scale up to a power of two (use_ue8m0=True of the quantisers), for the hardware-scaled GEMM.
template <int MODE>
__global__ void __launch_bounds__(256) quant_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                         float* __restrict__ sf, long long rows, int cols, int blocks_per_row,
                                                         int pow2_scales, const int* __restrict__ rows_limit) {
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = rows * blocks_per_row;
  if (warp_global >= total) return;
  const long long row = warp_global / blocks_per_row;
  if (rows_limit != nullptr && row >= *rows_limit) return;   // rows past the count the device holds are not touched
  const int blk = static_cast<int>(warp_global - row * blocks_per_row);
  const int c0 = blk * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  const int in_cols = MODE == 1 ? 2 * cols : cols;
  const __nv_bfloat16* xr = x + row * in_cols;
  if (c0 + 3 < cols) {
    const uint2 g = *reinterpret_cast<const uint2*>(xr + c0);
    const __nv_bfloat162 g0 = *reinterpret_cast<const __nv_bfloat162*>(&g.x), g1 = *reinterpret_cast<const __nv_bfloat162*>(&g.y);
    v[0] = __low2float(g0); v[1] = __high2float(g0); v[2] = __low2float(g1); v[3] = __high2float(g1);
    if (MODE == 1) {
      const uint2 u = *reinterpret_cast<const uint2*>(xr + cols + c0);
      const __nv_bfloat162 u0 = *reinterpret_cast<const __nv_bfloat162*>(&u.x), u1 = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
      const float uu[4] = {__low2float(u0), __high2float(u0), __low2float(u1), __high2float(u1)};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float s = v[i] / (1.0f + expf(-v[i]));
        v[i] = __bfloat162float(__float2bfloat16_rn(s * uu[i]));
      }
    }
  } else {
    for (int i = 0; i < 4; ++i) {
      if (c0 + i < cols) {
        float g = __bfloat162float(xr[c0 + i]);
        if (MODE == 1) {
          const float s = g / (1.0f + expf(-g));
          g = __bfloat162float(__float2bfloat16_rn(s * __bfloat162float(xr[cols + c0 + i])));
        }
        v[i] = g;
      }
    }
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = fmaxf(warp_max(amax), 1e-4f);
  float scale = amax * (1.0f / kFp8Max);  // torch's CUDA division by a scalar multiplies by its fp32 reciprocal
  if (pow2_scales) scale = ceil_pow2(scale);
  const float inv = 1.0f / scale;
  const uint32_t packed = quantise4(v, inv);
  uint8_t* qr = q + row * cols;
  if (c0 + 3 < cols) {
    *reinterpret_cast<uint32_t*>(qr + c0) = packed;
  } else {
    for (int i = 0; i < 4; ++i)
      if (c0 + i < cols) qr[c0 + i] = static_cast<uint8_t>(packed >> (8 * i));
  }
  if (lane == 0) sf[row * blocks_per_row + blk] = scale;
}

// Wide form of quant_rows_kernel for 16-byte aligned rows with cols % 8 == 0: one warp per (row, pair of 128-column
// blocks), each half-warp owns one block and each lane 8 consecutive columns (16-byte loads, 8-byte stores), so a warp
// keeps twice the bytes in flight. Per-element arithmetic and the scale are those of quant_rows_kernel, bit for bit.
template <int MODE>
__global__ void __launch_bounds__(256) quant_rows_wide_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                              float* __restrict__ sf, long long rows, int cols, int blocks_per_row,
                                                              int pairs_per_row, int pow2_scales, const int* __restrict__ rows_limit) {
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= rows * pairs_per_row) return;
  const long long row = warp_global / pairs_per_row;
  if (rows_limit != nullptr && row >= *rows_limit) return;
  const int pair = static_cast<int>(warp_global - row * pairs_per_row);
  const int blk = pair * 2 + (lane >> 4);
  const int c0 = blk * 128 + (lane & 15) * 8;
  const bool live = blk < blocks_per_row && c0 < cols;       // cols % 8 == 0: a lane's 8 columns are all in or all out
  const int in_cols = MODE == 1 ? 2 * cols : cols;
  const __nv_bfloat16* xr = x + row * in_cols;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) {
    const uint4 g = *reinterpret_cast<const uint4*>(xr + c0);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __low2float(gp[i]);
      v[2 * i + 1] = __high2float(gp[i]);
    }
    if (MODE == 1) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + cols + c0);
      const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float u0 = __low2float(up[i]), u1 = __high2float(up[i]);
        const float s0 = v[2 * i] / (1.0f + expf(-v[2 * i]));
        const float s1 = v[2 * i + 1] / (1.0f + expf(-v[2 * i + 1]));
        v[2 * i] = __bfloat162float(__float2bfloat16_rn(s0 * u0));
        v[2 * i + 1] = __bfloat162float(__float2bfloat16_rn(s1 * u1));
      }
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // within the half-warp
  amax = fmaxf(amax, 1e-4f);
  float scale = amax * (1.0f / kFp8Max);
  if (pow2_scales) scale = ceil_pow2(scale);
  const float inv = 1.0f / scale;
  if (live) {
    const float lo[4] = {v[0], v[1], v[2], v[3]}, hi[4] = {v[4], v[5], v[6], v[7]};
    uint2 packed;
    packed.x = quantise4(lo, inv);
    packed.y = quantise4(hi, inv);
    *reinterpret_cast<uint2*>(q + row * cols + c0) = packed;
  }
  if ((lane & 15) == 0 && blk < blocks_per_row) sf[row * blocks_per_row + blk] = scale;
}

// dst[dst_rows ? dst_rows[i] : i] = src[src_rows ? src_rows[i] : i] for i < rows; one warp per row, 16-byte vectors.
__global__ void __launch_bounds__(256) move_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                        const long long* __restrict__ src_rows, const long long* __restrict__ dst_rows,
                                                        long long rows, int vec_per_row) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= rows) return;
  const long long s = src_rows ? src_rows[w] : w;
  const long long d = dst_rows ? dst_rows[w] : w;
  const uint4* sp = src + s * vec_per_row;
  uint4* dp = dst + d * vec_per_row;
  for (int i = lane; i < vec_per_row; i += 32) dp[i] = sp[i];
}

// y[t] = sum_j w[t, j] * rows[pos[t * k + j]] in fp32, rounded once to bf16. One CTA per token, 8 columns per thread.
__global__ void __launch_bounds__(256) combine_topk_kernel(const __nv_bfloat16* __restrict__ rows, const long long* __restrict__ pos,
                                                           const float* __restrict__ w, __nv_bfloat16* __restrict__ y, int top_k, int cols) {
  const long long t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const long long r = pos != nullptr ? pos[t * top_k + j] : t * top_k + j;
      const float wt = w[t * top_k + j];
      const uint4 v = *reinterpret_cast<const uint4*>(rows + r * cols + c);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] = fmaf(wt, __low2float(p[i]), acc[2 * i]);
        acc[2 * i + 1] = fmaf(wt, __high2float(p[i]), acc[2 * i + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) op[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(y + t * cols + c) = o;
  }
}

// One warp per row: scale = max(amax(row) * (1/127), 1e-12), q = clamp(rint(x * (1 / scale)), -127, 127); the scale is written
// to every one of the row's `kb` K-block slots, which is how the reference feeds its per-token INT8 scales to the grouped
// GEMM (quantize_per_token_int8_gpu + expand, asym_gemm/unified_moe/runtime.py:573-583,1558-1562).
// MODE 0: x is bf16 [rows, cols]. MODE 1: x is fp32 [rows, 2*cols] = gate | up and the value quantised is
// bf16(silu(gate) * up) (runtime.py:1570,1620-1627).
template <int MODE>
__global__ void __launch_bounds__(256) quant_rows_int8_kernel(const void* __restrict__ xin, int8_t* __restrict__ q, float* __restrict__ sf,
                                                              long long rows, int cols, int kb) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  auto value = [&](int c) -> float {
    if (MODE == 0) return __bfloat162float(static_cast<const __nv_bfloat16*>(xin)[row * cols + c]);
    const float* g = static_cast<const float*>(xin) + row * 2 * cols;
    const float gate = g[c];
    return __bfloat162float(__float2bfloat16_rn((gate / (1.0f + expf(-gate))) * g[cols + c]));
  };
  float amax = 0.f;
  for (int c = lane; c < cols; c += 32) amax = fmaxf(amax, fabsf(value(c)));
  amax = warp_max(amax);
  const float scale = fmaxf(amax * (1.0f / 127.0f), 1e-12f);
  const float inv = 1.0f / scale;
  for (int c = lane; c < cols; c += 32) {
    const float r = fminf(fmaxf(rintf(value(c) * inv), -127.f), 127.f);
    q[row * cols + c] = static_cast<int8_t>(r);
  }
  for (int i = lane; i < kb; i += 32) sf[row * kb + i] = scale;
}

// fp32-row variant of combine_topk_kernel (the reference keeps the INT8 layer's down-projection output in fp32).
__global__ void __launch_bounds__(256) combine_topk_f32_kernel(const float* __restrict__ rows, const long long* __restrict__ pos,
                                                               const float* __restrict__ w, __nv_bfloat16* __restrict__ y, int top_k, int cols) {
  const long long t = blockIdx.x;
  for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const long long r = pos[t * top_k + j];
      const float wt = w[t * top_k + j];
      const float4 v = *reinterpret_cast<const float4*>(rows + r * cols + c);
      acc[0] = fmaf(wt, v.x, acc[0]); acc[1] = fmaf(wt, v.y, acc[1]); acc[2] = fmaf(wt, v.z, acc[2]); acc[3] = fmaf(wt, v.w, acc[3]);
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0], acc[1]), hi = __floats2bfloat162_rn(acc[2], acc[3]);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(y + t * cols + c) = o;
  }
}

}  // namespace agb

namespace {
int launch_check() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? AG_OK : agb_fail(AG_E_CUDA, cudaGetErrorString(e));
}
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
bool aligned_to(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
}  // namespace

extern "C" {

int ag_quant_rows_fp8_upto(const void* x_bf16, void* q, float* sf, int64_t rows, int64_t cols, int32_t pow2_scales, const int32_t* rows_used,
                           void* stream) {
  if (!x_bf16 || !q || !sf || rows < 0 || cols <= 0 || cols % 4 != 0) return agb_fail(AG_E_INVALID, "bad arguments (cols must be a multiple of 4)");
  if (rows == 0) return AG_OK;
  // the narrow kernel reads 8 bytes of x and writes 4 bytes of q per lane (the wide one 16 and 8)
  if (!aligned_to(x_bf16, 8) || !aligned_to(q, 4) || !aligned_to(sf, 4))
    return agb_fail(AG_E_INVALID, "x must be 8-byte aligned, q and sf 4-byte aligned");
  const int bpr = static_cast<int>((cols + 127) / 128);
  if (cols % 8 == 0 && aligned16(x_bf16) && (reinterpret_cast<uintptr_t>(q) & 7) == 0) {
    const int ppr = (bpr + 1) / 2;
    const long long wide = rows * ppr;
    agb::quant_rows_wide_kernel<0><<<static_cast<unsigned>((wide + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(q), sf, rows, static_cast<int>(cols), bpr, ppr, pow2_scales, rows_used);
    return launch_check();
  }
  const long long warps = rows * bpr;
  agb::quant_rows_kernel<0><<<static_cast<unsigned>((warps + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(q), sf, rows, static_cast<int>(cols), bpr, pow2_scales, rows_used);
  return launch_check();
}

int ag_quant_rows_fp8(const void* x_bf16, void* q, float* sf, int64_t rows, int64_t cols, int32_t pow2_scales, void* stream) {
  return ag_quant_rows_fp8_upto(x_bf16, q, sf, rows, cols, pow2_scales, nullptr, stream);
}

int ag_silu_mul_quant_fp8_upto(const void* gate_up_bf16, void* q, float* sf, int64_t rows, int64_t inter, int32_t pow2_scales,
                               const int32_t* rows_used, void* stream) {
  if (!gate_up_bf16 || !q || !sf || rows < 0 || inter <= 0 || inter % 4 != 0) return agb_fail(AG_E_INVALID, "bad arguments (inter must be a multiple of 4)");
  if (rows == 0) return AG_OK;
  if (!aligned_to(gate_up_bf16, 8) || !aligned_to(q, 4) || !aligned_to(sf, 4))
    return agb_fail(AG_E_INVALID, "gate_up must be 8-byte aligned, q and sf 4-byte aligned");
  const int bpr = static_cast<int>((inter + 127) / 128);
  if (inter % 8 == 0 && aligned16(gate_up_bf16) && (reinterpret_cast<uintptr_t>(q) & 7) == 0) {
    const int ppr = (bpr + 1) / 2;
    const long long wide = rows * ppr;
    agb::quant_rows_wide_kernel<1><<<static_cast<unsigned>((wide + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(gate_up_bf16), static_cast<uint8_t*>(q), sf, rows, static_cast<int>(inter), bpr, ppr, pow2_scales, rows_used);
    return launch_check();
  }
  const long long warps = rows * bpr;
  agb::quant_rows_kernel<1><<<static_cast<unsigned>((warps + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up_bf16), static_cast<uint8_t*>(q), sf, rows, static_cast<int>(inter), bpr, pow2_scales, rows_used);
  return launch_check();
}

int ag_silu_mul_quant_fp8(const void* gate_up_bf16, void* q, float* sf, int64_t rows, int64_t inter, int32_t pow2_scales, void* stream) {
  return ag_silu_mul_quant_fp8_upto(gate_up_bf16, q, sf, rows, inter, pow2_scales, nullptr, stream);
}

int ag_move_rows(const void* src, void* dst, const int64_t* src_rows, const int64_t* dst_rows, int64_t rows, int64_t row_bytes, void* stream) {
  if (!src || !dst || rows < 0 || row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(src) || !aligned16(dst))
    return agb_fail(AG_E_INVALID, "bad arguments (rows must be 16-byte multiples and 16-byte aligned)");
  if (rows == 0) return AG_OK;
  agb::move_rows_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), reinterpret_cast<const long long*>(src_rows),
      reinterpret_cast<const long long*>(dst_rows), rows, static_cast<int>(row_bytes / 16));
  return launch_check();
}

int ag_combine_topk(const void* rows_bf16, const int64_t* pos, const float* weights, void* y_bf16, int64_t tokens, int32_t top_k,
                    int64_t cols, void* stream) {
  if (!rows_bf16 || !weights || !y_bf16 || tokens < 0 || top_k <= 0 || cols <= 0 || cols % 8 != 0 || !aligned16(rows_bf16) ||
      !aligned16(y_bf16) || !aligned_to(pos, 8) || !aligned_to(weights, 4))
    return agb_fail(AG_E_INVALID, "bad arguments (cols must be a multiple of 8; rows and y 16-byte aligned)");
  if (tokens == 0) return AG_OK;
  agb::combine_topk_kernel<<<static_cast<unsigned>(tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(rows_bf16), reinterpret_cast<const long long*>(pos), weights, static_cast<__nv_bfloat16*>(y_bf16),
      top_k, static_cast<int>(cols));
  return launch_check();
}

int ag_quant_rows_int8(const void* x_bf16, void* q, float* sf, int64_t rows, int64_t cols, void* stream) {
  if (!x_bf16 || !q || !sf || rows < 0 || cols <= 0 || !aligned_to(x_bf16, 2) || !aligned_to(sf, 4))
    return agb_fail(AG_E_INVALID, "bad arguments (x must be 2-byte aligned, sf 4-byte aligned)");
  if (rows == 0) return AG_OK;
  agb::quant_rows_int8_kernel<0><<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x_bf16, static_cast<int8_t*>(q), sf, rows, static_cast<int>(cols), static_cast<int>((cols + 127) / 128));
  return launch_check();
}

int ag_silu_mul_quant_int8(const void* gate_up_f32, void* q, float* sf, int64_t rows, int64_t inter, void* stream) {
  if (!gate_up_f32 || !q || !sf || rows < 0 || inter <= 0 || !aligned_to(gate_up_f32, 4) || !aligned_to(sf, 4))
    return agb_fail(AG_E_INVALID, "bad arguments (gate_up and sf must be 4-byte aligned)");
  if (rows == 0) return AG_OK;
  agb::quant_rows_int8_kernel<1><<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      gate_up_f32, static_cast<int8_t*>(q), sf, rows, static_cast<int>(inter), static_cast<int>((inter + 127) / 128));
  return launch_check();
}

int ag_combine_topk_f32(const void* rows_f32, const int64_t* pos, const float* weights, void* y_bf16, int64_t tokens, int32_t top_k,
                        int64_t cols, void* stream) {
  if (!rows_f32 || !pos || !weights || !y_bf16 || tokens < 0 || top_k <= 0 || cols <= 0 || cols % 4 != 0 || !aligned16(rows_f32) ||
      !aligned_to(y_bf16, 8) || !aligned_to(pos, 8) || !aligned_to(weights, 4))
    return agb_fail(AG_E_INVALID, "bad arguments (cols must be a multiple of 4; rows 16-byte and y 8-byte aligned)");
  if (tokens == 0) return AG_OK;
  agb::combine_topk_f32_kernel<<<static_cast<unsigned>(tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(rows_f32), reinterpret_cast<const long long*>(pos), weights, static_cast<__nv_bfloat16*>(y_bf16), top_k,
      static_cast<int>(cols));
  return launch_check();
}

}  // extern "C"
