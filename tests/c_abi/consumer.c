/* A plain-C user of the library: proves that include/asymgemm_b200.h compiles as C (no C++ in the interface), that a
 * program links against the shared library with nothing but the header, and that the entry points answer malformed
 * requests with an error code and a message instead of touching a GPU. Built and run by tests/test_host_logic.py. */
#include <stdio.h>
#include <string.h>

#include "asymgemm_b200.h"

static int expect(int cond, const char* what) {
  if (!cond) fprintf(stderr, "FAILED: %s (last error: %s)\n", what, ag_last_error());
  return cond ? 0 : 1;
}

int main(void) {
  int bad = 0;
  ag_gemm_desc_t g;
  memset(&g, 0, sizeof(g));

  bad += expect(ag_version() != NULL && strlen(ag_version()) > 0, "ag_version returns a string");
  bad += expect(ag_get_mk_alignment_for_contiguous_layout() == 128, "contiguous-layout alignment is 128");
  bad += expect(ag_gemm_desc_size() == sizeof(ag_gemm_desc_t), "the library and this program agree on the descriptor");
  bad += expect(ag_m_grouped_bf16_gemm_nt(NULL) == AG_E_INVALID, "NULL descriptor is refused");
  bad += expect(strstr(ag_last_error(), "desc") != NULL, "the message names the descriptor");

  g.layout = 7;
  g.n = 256; g.k = 512; g.num_groups = 2; g.m = 128;
  bad += expect(ag_m_grouped_fp8_gemm_nt(&g) == AG_E_INVALID, "unknown layout is refused");
  g.layout = AG_LAYOUT_CONTIGUOUS;
  g.n = 0;
  bad += expect(ag_m_grouped_int8_gemm_nt(&g) == AG_E_INVALID, "n = 0 is refused");
  g.n = 256;
  g.m = 0;
  bad += expect(ag_m_grouped_fp4_gemm_nt(&g) == AG_OK, "an empty problem is a no-op");

  /* sizes are pure arithmetic: no device needed */
  bad += expect(ag_scratch_bytes(1, 4096, 7168, 148) > 0, "scratch size for the FP8 kernel");
  bad += expect(ag_fp4_sf_blocked_bytes(1, 128, 256) == ag_fp4_sf_blocked_bytes(2, 128, 256) / 2, "blocked scale bytes scale with groups");
  bad += expect(ag_static_scratch_bytes() >= (64u << 20), "the built-in scratch is tens of MiB");
  bad += expect(ag_release_weights(&g) == AG_E_INVALID, "releasing memory that was never prepared is refused");

  ag_set_num_sms(100);
  bad += expect(ag_get_num_sms() == 100, "num_sms round trip");
  ag_set_num_sms(0);

  if (bad == 0) printf("c_abi consumer: ok (%s)\n", ag_version());
  return bad;
}
