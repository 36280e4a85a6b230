/* A plain C caller of the C-ABI, the way the reference's test/tools/runtime/test_capi_runtime.cpp uses it:
 * handles, error convention (status 0/1, message in the caller's buffer, buffer untouched on success), and - with a
 * device - compile a launch descriptor, run it through afirt_executor_run and afirt_executor_run_file on host
 * arrays and memcmp the result with the expectation computed here.
 *   test_capi_runtime cpu                       no device needed
 *   test_capi_runtime gpu <descriptor.json> <work dir>
 * Compiled as C99 against include/CAPI/Runtime.h only, linked with -lAFIRRuntimeCAPI.  Exit code = failed checks. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "CAPI/Runtime.h"

static int g_pass = 0, g_fail = 0;
#define EXPECT(cond, what)                                                        \
  do {                                                                            \
    if (cond) ++g_pass;                                                           \
    else { ++g_fail; fprintf(stderr, "FAIL: %s (line %d)\n", what, __LINE__); }   \
  } while (0)

static void put_i64(uint8_t *dst, long long v) {
  int i;
  for (i = 0; i < 8; ++i) dst[i] = (uint8_t)(((unsigned long long)v >> (8 * i)) & 0xff);
}

static void check_error_convention(void) {
  char err[256];
  float x = 1.0f, y = 0.0f;
  const void *ins[1] = {&x};
  void *outs[1] = {&y};
  size_t in_bytes[1] = {sizeof x}, out_bytes[1] = {sizeof y};
  const uint8_t binary[4] = {1, 2, 3, 4};
  AfirtExecutor exe = afirt_executor_create();
  AfirtCompiler cc = afirt_compiler_create("sm_100a", "sm_100a", 3);
  EXPECT(exe != NULL && cc != NULL, "handles are created");

  memset(err, 0, sizeof err);
  EXPECT(afirt_executor_run(exe, binary, sizeof binary, "k", 1, ins, in_bytes, 1, outs, out_bytes, NULL, 0, 1, 0x41415246u, err,
                            sizeof err) != 0 && strstr(err, "executor has not been initialized") != NULL,
         "run before initialize is refused with the reference's message");
  memset(err, 0, sizeof err);
  EXPECT(afirt_executor_initialize(exe, -1, err, sizeof err) != 0 && err[0] != '\0', "negative device id is refused");
  memset(err, 0, sizeof err);
  EXPECT(afirt_executor_run_file(exe, "/nonexistent/kernel.bin", "k", 1, ins, in_bytes, 1, outs, out_bytes, NULL, 0, 1, 0x41415246u,
                                 err, sizeof err) != 0 && err[0] != '\0',
         "missing binary file is an error");
  {
    char small[8];
    memset(small, 'x', sizeof small);
    EXPECT(afirt_executor_initialize(exe, -1, small, sizeof small) != 0 && small[sizeof small - 1] == '\0',
           "messages are truncated to the buffer and NUL-terminated");
  }
  {
    char path[512];
    memset(path, 0, sizeof path);
    EXPECT(afirt_compiler_compile(cc, "/nonexistent/kernel.cuda.json", "/tmp", "k", path, sizeof path) != 0 && path[0] != '\0',
           "compile of a missing source reports through the path buffer");
  }
  afirt_compiler_destroy(cc);
  afirt_executor_destroy(exe);
  afirt_compiler_destroy(NULL);
  afirt_executor_destroy(NULL);
  ++g_pass; /* destroying NULL handles did not crash */
}

static void check_device_run(const char *descriptor, const char *workdir) {
  enum { M = 37, N = 300 };
  static float a[M * N], b[M * N], got[M * N], want[M * N];
  char err[512], bin_path[1024];
  uint8_t tiling[4 * 8];
  const void *ins[2];
  void *outs[1];
  size_t in_bytes[2], out_bytes[1];
  unsigned s = 12345u;
  int i;
  AfirtCompiler cc = afirt_compiler_create("sm_100a", "sm_100a", 3);
  AfirtExecutor exe = afirt_executor_create();
  for (i = 0; i < M * N; ++i) {
    volatile float sum;
    s = s * 1664525u + 1013904223u;
    a[i] = (float)(s >> 8) / 8388608.0f - 1.0f;
    s = s * 1664525u + 1013904223u;
    b[i] = (float)(s >> 8) / 8388608.0f - 1.0f;
    sum = a[i] + b[i]; /* rounded to f32 before the multiply: no contraction */
    want[i] = sum * b[i];
  }
  memset(bin_path, 0, sizeof bin_path);
  EXPECT(afirt_compiler_compile(cc, descriptor, workdir, "add_mul", bin_path, sizeof bin_path) == 0, "descriptor compiles");
  memset(err, 0, sizeof err);
  EXPECT(afirt_executor_initialize(exe, 0, err, sizeof err) == 0 && err[0] == '\0', "device 0 initialises, buffer untouched");
  /* TilingData: CTA_THREADS, UNROLL, dim_arg0_0, dim_arg0_1 as little-endian int64 */
  put_i64(tiling + 0, 128);
  put_i64(tiling + 8, 2);
  put_i64(tiling + 16, M);
  put_i64(tiling + 24, N);
  ins[0] = a; ins[1] = b; outs[0] = got;
  in_bytes[0] = in_bytes[1] = out_bytes[0] = sizeof a;
  memset(err, 'z', sizeof err);
  memset(got, 0, sizeof got);
  EXPECT(afirt_executor_run_file(exe, bin_path, "add_mul", 2, ins, in_bytes, 1, outs, out_bytes, tiling, sizeof tiling, 0, 0x41415246u,
                                 err, sizeof err) == 0, "run_file succeeds");
  EXPECT(err[0] == 'z' && err[1] == 'z', "error buffer untouched on success");
  EXPECT(memcmp(got, want, sizeof want) == 0, "run_file result equals the expectation bit for bit");
  {
    FILE *f = fopen(bin_path, "rb");
    static uint8_t binary[1 << 16];
    size_t n = f ? fread(binary, 1, sizeof binary, f) : 0;
    if (f) fclose(f);
    memset(got, 0, sizeof got);
    memset(err, 0, sizeof err);
    EXPECT(n > 0 && afirt_executor_run(exe, binary, n, "add_mul", 2, ins, in_bytes, 1, outs, out_bytes, tiling, sizeof tiling, 0,
                                       0x41415246u, err, sizeof err) == 0 && memcmp(got, want, sizeof want) == 0,
           "run from memory gives the same bytes");
    memset(err, 0, sizeof err);
    EXPECT(afirt_executor_run(exe, binary, n, "add_mul", 2, ins, in_bytes, 1, outs, out_bytes, tiling, sizeof tiling, 0, 0x12345678u, err,
                              sizeof err) != 0 && strstr(err, "unsupported kernel magic") != NULL,
           "unknown magic is refused");
    memset(err, 0, sizeof err);
    in_bytes[1] = sizeof a - 4;
    EXPECT(afirt_executor_run(exe, binary, n, "add_mul", 2, ins, in_bytes, 1, outs, out_bytes, tiling, sizeof tiling, 0, 0x41415246u, err,
                              sizeof err) != 0 && strstr(err, "[cuda:bindings]") != NULL,
           "a byte count that contradicts the shape is a bindings error");
  }
  afirt_executor_destroy(exe);
  afirt_compiler_destroy(cc);
}

int main(int argc, char **argv) {
  if (argc >= 2 && strcmp(argv[1], "cpu") == 0) check_error_convention();
  else if (argc >= 4 && strcmp(argv[1], "gpu") == 0) { check_error_convention(); check_device_run(argv[2], argv[3]); }
  else { fprintf(stderr, "usage: %s cpu | gpu <descriptor.json> <work dir>\n", argv[0]); return 2; }
  printf("%d passed, %d failed\n", g_pass, g_fail);
  return g_fail;
}
