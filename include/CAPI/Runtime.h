/* libAFIRRuntimeCAPI.so -- C entry points of the B200 runtime.
 *
 * These seven functions keep the names, argument lists and error convention of the
 * Ascend-MLIR runtime C API (reference include/CAPI/Runtime.h:17-102, implemented in
 * lib/CAPI/Runtime/Runtime.cpp:306-481) so that its callers -- python/runtime/executor.py,
 * python/runtime/compiler.py and test/tools/runtime/test_capi_runtime.cpp -- bind unchanged.
 *
 * Conventions (all from the reference implementation):
 *  - handles are opaque heap objects, created and destroyed in pairs; the caller owns them;
 *  - tensors are HOST pointers owned by the caller, outputs pre-allocated and filled on return;
 *  - int results: 0 = success, non-zero = failure with a NUL-terminated, truncated message in
 *    the caller's buffer; on success the buffer is left untouched;
 *  - a handle is not internally locked: one thread per handle at a time.
 *
 * What differs underneath: the "kernel source" handed to the compiler is the launch descriptor
 * written by `afir-translate -mlir-to-cuda`, the "binary" is that descriptor sealed in a small
 * container, and execution launches the matching hand-written sm_100a kernel of this library on
 * a CUDA device instead of an AscendC ELF on the CANN simulator.
 */
#ifndef AFIR_CAPI_RUNTIME_H
#define AFIR_CAPI_RUNTIME_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct AfirtCompiler_s *AfirtCompiler;
typedef struct AfirtExecutor_s *AfirtExecutor;

/* Replaces afirt_compiler_create (reference include/CAPI/Runtime.h:29-31).
 * soc_version: informational ("sm_100a" or an Ascend SoC name, kept for callers that pass one).
 * arch: "sm_100a", or the reference's "dav-c220-vec" / "dav-c220-cube" (accepted and mapped).
 * Returns NULL only on allocation failure. */
AfirtCompiler afirt_compiler_create(const char *soc_version, const char *arch, int opt_level);

/* Replaces afirt_compiler_destroy (reference include/CAPI/Runtime.h:33). */
void afirt_compiler_destroy(AfirtCompiler compiler);

/* Replaces afirt_compiler_compile (reference include/CAPI/Runtime.h:39-44):
 * src_file -> output_dir/kernel_name.bin.  Validates the launch descriptor against the kernel
 * library, writes the container and an output_dir/manifest.txt (kernel_name, soc_version,
 * kernel_kind, device_binary_path, manifest_path).  On success out_bin_path receives the path;
 * on failure it receives the error text. */
int afirt_compiler_compile(AfirtCompiler compiler, const char *src_file, const char *output_dir,
                           const char *kernel_name, char *out_bin_path, size_t buf_len);

/* Replace afirt_executor_create / afirt_executor_destroy (reference include/CAPI/Runtime.h:52-53). */
AfirtExecutor afirt_executor_create(void);
void afirt_executor_destroy(AfirtExecutor executor);

/* Replaces afirt_executor_initialize (reference include/CAPI/Runtime.h:57-58).
 * Records the CUDA device ordinal; device_id < 0 is an error. */
int afirt_executor_initialize(AfirtExecutor executor, int device_id, char *err_buf, size_t err_len);

/* Replaces afirt_executor_run (reference include/CAPI/Runtime.h:75-86).
 *   binary_data/binary_len : kernel container (or bare descriptor JSON)
 *   function_name          : kernel entry point; must be the one the binary defines
 *   input_ptrs/input_bytes : num_inputs host tensors, flat
 *   output_ptrs/output_bytes: num_outputs pre-allocated host buffers
 *   tiling_data/tiling_len : packed TilingData, little-endian, schema order
 *   block_dim              : number of thread blocks (<= 0: library default)
 *   magic                  : 0x41415246 (vector/mixed) or 0x41494343 (cube); others are refused
 * Copies inputs to the device, launches, waits, copies outputs back. */
int afirt_executor_run(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                       const char *function_name, int num_inputs, const void **input_ptrs,
                       const size_t *input_bytes, int num_outputs, void **output_ptrs,
                       const size_t *output_bytes, const uint8_t *tiling_data, size_t tiling_len,
                       int block_dim, uint32_t magic, char *err_buf, size_t err_len);

/* Replaces afirt_executor_run_file (reference include/CAPI/Runtime.h:89-100): reads the binary
 * from binary_path, then behaves as afirt_executor_run. */
int afirt_executor_run_file(AfirtExecutor executor, const char *binary_path, const char *function_name,
                            int num_inputs, const void **input_ptrs, const size_t *input_bytes,
                            int num_outputs, void **output_ptrs, const size_t *output_bytes,
                            const uint8_t *tiling_data, size_t tiling_len, int block_dim,
                            uint32_t magic, char *err_buf, size_t err_len);

#ifdef __cplusplus
}
#endif

#endif /* AFIR_CAPI_RUNTIME_H */
