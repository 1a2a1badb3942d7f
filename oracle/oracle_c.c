/*
 * Plain-C restatement of the grouped GEMM arithmetic -- TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline;
 * never linked into or called by the product).
 *
 * ago_int8_grouped follows the reference's INT8 semantics: an exact int32 dot product per 128-wide K block, scaled by
 * sfa[row, kb] * sfb[col, kb] in fp32 and summed over K blocks in ascending order
 * (asym_gemm/include/asym_gemm/impls/sm90_int8_asym_gemm_1d1d.cuh:347-353,439-447; scalar reference of the CPU
 * library: csrc/cpu/cpu_gemm/tests/reference.h:98-124).
 * ago_f32_grouped is the per-expert `a[s:e] @ w.t()` loop of the reference's torch CPU path
 * (asym_gemm/training/frozen_linear.py:986-1008) on operands the caller has already dequantised to fp32.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* segments: n_seg triples (expert, row_start, row_end). */
void ago_int8_grouped(const int8_t* a, const float* sfa, const int8_t* b, const float* sfb, float* d, int32_t* block_sums,
                      const int32_t* segments, int n_seg, long rows_total, long n, long k) {
  const long kb = (k + 127) / 128;
  for (int s = 0; s < n_seg; ++s) {
    const long e = segments[3 * s], r0 = segments[3 * s + 1], r1 = segments[3 * s + 2];
    for (long r = r0; r < r1; ++r) {
      const int8_t* ar = a + r * k;
      for (long c = 0; c < n; ++c) {
        const int8_t* bc = b + (e * n + c) * k;
        float acc = 0.f;
        for (long i = 0; i < kb; ++i) {
          const long k0 = i * 128, k1 = k0 + 128 < k ? k0 + 128 : k;
          int32_t sum = 0;
          for (long j = k0; j < k1; ++j) sum += (int32_t)ar[j] * (int32_t)bc[j];
          if (block_sums) block_sums[(i * rows_total + r) * n + c] = sum;
          acc = (float)sum * (sfa[r * kb + i] * sfb[(e * n + c) * kb + i]) + acc;
        }
        d[r * n + c] = acc;
      }
    }
  }
}

void ago_f32_grouped(const float* a, const float* b, float* d, const int32_t* segments, int n_seg, long n, long k) {
  for (int s = 0; s < n_seg; ++s) {
    const long e = segments[3 * s], r0 = segments[3 * s + 1], r1 = segments[3 * s + 2];
    for (long r = r0; r < r1; ++r) {
      for (long c = 0; c < n; ++c) {
        const float* ar = a + r * k;
        const float* bc = b + (e * n + c) * k;
        float acc = 0.f;
        for (long j = 0; j < k; ++j) acc += ar[j] * bc[j];
        d[r * n + c] = acc;
      }
    }
  }
}
