/* A plain-C client of the library: includes only include/falkon_b200.h, links against libfalkon_b200.so and
 * exercises the entry points that need no GPU (version, status names, workspace arithmetic, argument checks).
 * Built and run by tests/test_abi.py::test_plain_c_client. */
#include <stdio.h>
#include <string.h>

#include "falkon_b200.h"

int main(void) {
  int failures = 0;
  if (flk_version() < 100) { printf("bad version\n"); ++failures; }
  if (strcmp(flk_status_name(FLK_ERR_WORKSPACE), "FLK_ERR_WORKSPACE") != 0) { printf("bad status name\n"); ++failures; }
  /* benchmark configuration 3: N = 1e7, d = 28, M = 50000, T = 1, fp32 Gaussian */
  int64_t need = flk_fdmmv_workspace_bytes(FLK_F32, FLK_GAUSSIAN, 10000000, 50000, 28, 1, 0);
  if (need <= 0 || need > ((int64_t)16 << 30)) { printf("unexpected workspace size %lld\n", (long long)need); ++failures; }
  if (flk_fdmmv_workspace_bytes(FLK_F32, FLK_GAUSSIAN, -1, 50000, 28, 1, 0) != FLK_ERR_BAD_ARG) { printf("negative n accepted\n"); ++failures; }
  if (!flk_uses_tensor_cores(FLK_F32, FLK_MATERN25, 28, 1, 0) || flk_uses_tensor_cores(FLK_F64, FLK_GAUSSIAN, 9, 1, 0)) {
    printf("unexpected kernel choice\n");
    ++failures;
  }
  /* a call with a null X1 must come back with a status code and a message, without touching a device */
  double sigma = 1.0;
  int st = flk_fmmv(FLK_F32, FLK_GAUSSIAN, NULL, 10, 4, 1, (const void*)4096, 5, 4, 1, 4, (const void*)4096, 1, 1, 1,
                    (void*)4096, 1, 1, &sigma, 1, (void*)4096, (int64_t)1 << 30, 0, NULL);
  if (st != FLK_ERR_BAD_ARG || strstr(flk_last_error(), "X1") == NULL) { printf("null X1: status %d, '%s'\n", st, flk_last_error()); ++failures; }
  printf(failures ? "FAILED\n" : "ok %lld\n", (long long)need);
  return failures;
}
