// Scale-factor re-layout for NVFP4: row-major UE4M3 bytes [groups, rows, k16] -> the blocked form that tcgen05.cp
// copies into TMEM. Takes the place of the reference's per-call byte repack
// (get_mn_major_tma_aligned_packed_byte_sf_tensor, csrc/apis/layout.hpp:14-35), with a different target layout.
//
// Blocked layout: [group][row tile of 128][k4][512 bytes], k4 = index of a run of 4 scales (64 elements of K),
// padded with zeros to a multiple of 32 runs; inside a block byte (r % 32) * 16 + ((r % 128) / 32) * 4 + c.
// The source may be pinned host memory: the kernel then reads it over the host link once.
#include <cuda_runtime.h>
#include <cstdint>

namespace agb {

__host__ __device__ inline long long fp4_sf_k4_padded(long long k16) { return ((k16 + 3) / 4 + 31) / 32 * 32; }

__global__ void fp4_sf_to_blocked_kernel(const uint8_t* __restrict__ src, uint32_t* __restrict__ dst, long long groups,
                                         long long rows, long long k16, long long row_tiles, long long k4p) {
  const long long total_words = groups * row_tiles * k4p * 128;  // 128 words of 4 bytes per block
  for (long long w = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; w < total_words;
       w += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int in_block = static_cast<int>(w & 127);
    const long long block = w >> 7;
    const long long k4 = block % k4p;
    const long long tile = (block / k4p) % row_tiles;
    const long long g = block / (k4p * row_tiles);
    const int lane = in_block >> 2;   // r % 32
    const int quarter = in_block & 3; // (r % 128) / 32
    const long long r = tile * 128 + quarter * 32 + lane;
    uint32_t v = 0;
    if (r < rows) {
      const uint8_t* s = src + (g * rows + r) * k16 + k4 * 4;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (k4 * 4 + c < k16) v |= static_cast<uint32_t>(s[c]) << (8 * c);
    }
    dst[w] = v;
  }
}

cudaError_t fp4_sf_to_blocked(const void* src, void* dst, long long groups, long long rows, long long k16, cudaStream_t stream) {
  const long long row_tiles = (rows + 127) / 128;
  const long long k4p = fp4_sf_k4_padded(k16);
  const long long total_words = groups * row_tiles * k4p * 128;
  if (total_words == 0) return cudaSuccess;
  long long blocks = (total_words + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  fp4_sf_to_blocked_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const uint8_t*>(src), static_cast<uint32_t*>(dst),
                                                                             groups, rows, k16, row_tiles, k4p);
  return cudaGetLastError();
}

// fp32 scales -> UE8M0 exponent bytes (bits 23..30, mantissa dropped: exact for powers of two, the truncation of
// asym_gemm/include/asym_gemm/impls/smxx_layout.cuh:96-100 otherwise) in the same blocked form: [group][row tile of 128]
// [k4 = kb / 4, padded to a multiple of 8][512 bytes], byte (r % 32) * 16 + ((r % 128) / 32) * 4 + kb % 4.
// src is [groups, ceil(rows / rows_per_scale), kb]; rows_per_scale = 1 for activations, 128 for 128x128 weight blocks.
__host__ __device__ inline long long fp8_sf_k4_padded(long long kb) { return ((kb + 3) / 4 + 7) / 8 * 8; }

__global__ void fp8_sf_to_blocked_ue8m0_kernel(const float* __restrict__ src, uint32_t* __restrict__ dst, long long groups, long long rows,
                                               long long kb, int rows_per_scale, long long row_tiles, long long k4p) {
  const long long src_rows = (rows + rows_per_scale - 1) / rows_per_scale;
  const long long total_words = groups * row_tiles * k4p * 128;
  for (long long w = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; w < total_words;
       w += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int in_block = static_cast<int>(w & 127);
    const long long block = w >> 7;
    const long long k4 = block % k4p;
    const long long tile = (block / k4p) % row_tiles;
    const long long g = block / (k4p * row_tiles);
    const long long r = tile * 128 + (in_block & 3) * 32 + (in_block >> 2);
    uint32_t v = 0;
    if (r < rows) {
      const float* s = src + (g * src_rows + r / rows_per_scale) * kb + k4 * 4;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (k4 * 4 + c < kb) v |= ((__float_as_uint(s[c]) >> 23) & 0xFFu) << (8 * c);
    }
    dst[w] = v;
  }
}

cudaError_t fp8_sf_to_blocked_ue8m0(const float* src, void* dst, long long groups, long long rows, long long kb, int rows_per_scale,
                                    cudaStream_t stream) {
  const long long row_tiles = (rows + 127) / 128;
  const long long k4p = fp8_sf_k4_padded(kb);
  const long long total_words = groups * row_tiles * k4p * 128;
  if (total_words == 0) return cudaSuccess;
  long long blocks = (total_words + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  fp8_sf_to_blocked_ue8m0_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, static_cast<uint32_t*>(dst), groups, rows, kb,
                                                                                    rows_per_scale, row_tiles, k4p);
  return cudaGetLastError();
}
long long fp8_sf_k4_padded_host(long long kb) { return fp8_sf_k4_padded(kb); }

long long fp4_sf_k4_padded_host(long long k16) { return fp4_sf_k4_padded(k16); }

}  // namespace agb
