/* Device-resident entry points of libAFIRRuntimeCAPI.so.
 *
 * The reference runtime keeps tensors on the device only inside one call
 * (lib/Runtime/Execution/NativeExecutionRunner.cpp:372-511 allocates, copies in, launches, copies
 * out and frees).  Callers that already hold their tensors in GPU memory use the functions below
 * to reach the same kernels without the host round trip; everything else (binary, function name,
 * TilingData, block_dim, magic, error convention) is as in CAPI/Runtime.h.
 */
#ifndef AFIR_CAPI_RUNTIME_CUDA_H
#define AFIR_CAPI_RUNTIME_CUDA_H

#include "CAPI/Runtime.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The launch half of NativeExecutionRunner::runWithHandle (reference
 * lib/Runtime/Execution/NativeExecutionRunner.cpp:436-476: argument list
 * [inputs..., outputs..., workspace, tiling] then rtKernelLaunch).  input_ptrs/output_ptrs are
 * DEVICE pointers on the executor's device.  workspace may be NULL (the executor then owns one;
 * that path may allocate) or a device buffer of workspace_bytes.  cuda_stream is a cudaStream_t
 * (NULL = default stream).  Returns after enqueueing; nothing is synchronised. */
int afirt_executor_launch_device(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                 const char *function_name, int num_inputs, const void **input_ptrs,
                                 const size_t *input_bytes, int num_outputs, void **output_ptrs,
                                 const size_t *output_bytes, const uint8_t *tiling_data, size_t tiling_len,
                                 int block_dim, uint32_t magic, void *workspace, size_t workspace_bytes,
                                 void *cuda_stream, char *err_buf, size_t err_len);

/* The wait half (reference NativeExecutionRunner.cpp:484-489, rtStreamSynchronize failure is an
 * error): waits for cuda_stream (NULL = the executor's own stream, or the device) and reports
 * device-side status words (gather index out of range, bounded-wait timeout in the matmul). */
int afirt_executor_synchronize(AfirtExecutor executor, void *cuda_stream, char *err_buf, size_t err_len);

/* Scratch bytes afirt_executor_launch_device needs for this binary at these tiling values
 * (the reference sizes the workspace per task, include/Runtime/Execution/TaskGraph.h:54). */
int afirt_executor_workspace_bytes(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                   const uint8_t *tiling_data, size_t tiling_len, size_t *out_bytes,
                                   char *err_buf, size_t err_len);

/* Kernels launched by the most recent run / launch on this executor, and since creation
 * (the launch counters the reference keeps per session, lib/Runtime/Execution/ExecutionSession.cpp:191-199). */
int afirt_executor_last_launch_count(AfirtExecutor executor);
uint64_t afirt_executor_total_launch_count(AfirtExecutor executor);

/* 1 when the most recent run / launch on this executor ran the group's GENERATED kernel -- the CUDA source that
 * afirt_compiler_compile (or, for a bare descriptor, the executor on first use) produced for that fused group and
 * compiled for sm_100a, loaded with cuModuleLoadData and started with cuLaunchKernel as
 * <kernel>(inputs..., outputs..., workspace, TilingData), the reference's kernel signature
 * (lib/Conversion/CanonicalizeCannSignature/CanonicalizeCannSignaturePass.cpp:57-140; registration and launch in
 * lib/Runtime/Execution/NativeExecutionRunner.cpp:223,476) -- and 0 when it ran a prebuilt kernel of the library
 * (matmul, bare transposes, and whatever AFIR_CUDA_CODEGEN = never | auto keeps there). */
int afirt_executor_last_launch_generated(AfirtExecutor executor);

/* No counterpart in the reference (its runtime allocates on every call).
 * out[m] = sum_n (a[m] + b[m,n]) with each row cut into split_cols column slices, for callers that
 * must not allocate GPU memory when they call: serving or real-time loops with a frozen memory
 * budget, processes whose device memory is fully committed, plugins under an allocator-owning framework.  The per-slice partial sums
 * live in a 1 MiB array built into the library (AFIRT_NO_ALLOC_MAX_PARTIALS floats per device)
 * instead of an allocated workspace; nothing here calls cudaMalloc, cudaFree or an allocating
 * library routine.  a [rows], b [rows, cols] and out [rows] are DEVICE pointers of elem_type
 * (0 = f32, 1 = f16, 2 = bf16); f32 accumulation.  rows * split_cols above the maximum is refused
 * with a message.  The first call on a device resolves the array's device address: make it before
 * any stream capture begins.  Every call on a device shares the array (contents left over from
 * the previous call are harmless: each call writes every slot it later reads), so calls that
 * overlap on the GPU race and must be serialised by the caller.  The call makes device_id current
 * for the launch and puts the caller's current device back before it returns.  Enqueues on
 * cuda_stream and returns; 0 = success, otherwise 1 with a message in err_buf. */
#define AFIRT_NO_ALLOC_MAX_PARTIALS 262144
int afirt_bcast_add_rowsum_no_alloc(int device_id, int elem_type, const void *a, const void *b, void *out,
                                    int64_t rows, int64_t cols, int split_cols, void *cuda_stream,
                                    char *err_buf, size_t err_len);

/* No counterpart in the reference (it runs on one device).  The row reduction with its REDUCED axis sharded
 * over the GPUs of one node: rank r holds the column slice b_r [rows, cols_r] and every rank wants
 *     out[m] = sum over ranks r of sum_n (a[m] + b_r[m, n]).
 * One kernel per rank does the local reduction and the exchange: each row's partial sum is stored straight
 * into every rank's mailbox over NVLink (peer-mapped memory) as one 8-byte entry {f32 sum, call number}, so
 * the value and the fact that it has arrived travel in the same store; the warp that sent a row picks up the
 * other ranks' entries a few rows later, a group of rows at a time with one lane per entry (waiting 2 s at
 * most), and adds them in rank order, so every rank ends with the same bits.  No flags, no fences, no library
 * collective.  (Few or short rows take the kernel without the staged stream; there the last CTA to finish
 * reads all rows.)  The call number lives in the mailbox and the kernel advances it itself, so a launch has no
 * argument that changes from call to call: a stream capture of these calls can be replayed as a CUDA graph, as
 * long as every rank replays the same number of calls.
 *
 *   create   allocates this rank's mailbox on device_id (2 x world_size x max_rows entries of 8 bytes) and
 *            writes AFIRT_EXCHANGE_HANDLE_BYTES bytes describing it to out_handle;
 *   connect  takes all ranks' handles in rank order (world_size x AFIRT_EXCHANGE_HANDLE_BYTES bytes, gathered
 *            by the caller over any transport) and maps the peers' mailboxes: CUDA IPC between processes,
 *            peer access inside one process;
 *   the reduction call enqueues the kernel on cuda_stream and returns.  a [rows], b [rows, cols] with
 *            b_row_stride elements between rows, out [rows] are DEVICE pointers of elem_type (0 f32, 1 f16,
 *            2 bf16).  It is collective: every rank makes the same sequence of calls with the same rows, and
 *            one rank's calls are ordered on one stream.  world_size 1 is allowed (a mailbox to itself);
 *   status   after the stream has been synchronised: 0, or 1 with a message when a wait ran out (the
 *            mailbox is then reset and can be used again once every rank has seen the failure);
 *   destroy  unmaps and frees; the caller makes sure no peer is still sending (a barrier).
 * Every rank needs its own GPU: ranks that wait for one another must never share a device. */
typedef struct AfirtRowsumExchange_s *AfirtRowsumExchange;
#define AFIRT_EXCHANGE_HANDLE_BYTES 96
#define AFIRT_EXCHANGE_MAX_RANKS 8
int afirt_rowsum_exchange_create(int device_id, int rank, int world_size, int64_t max_rows,
                                 AfirtRowsumExchange *out_exchange, uint8_t *out_handle, char *err_buf, size_t err_len);
int afirt_rowsum_exchange_connect(AfirtRowsumExchange exchange, const uint8_t *all_handles, char *err_buf, size_t err_len);
int afirt_bcast_add_rowsum_exchange(AfirtRowsumExchange exchange, int elem_type, const void *a, const void *b, void *out,
                                    int64_t rows, int64_t cols, int64_t b_row_stride, void *cuda_stream,
                                    char *err_buf, size_t err_len);
/* `count` independent reductions of one shape (a[i], b[i], out[i]) enqueued back to back by one call, for callers
 * with a queue of work; collective like the single call (every rank passes the same count).  No counterpart in
 * the reference. */
int afirt_bcast_add_rowsum_exchange_batch(AfirtRowsumExchange exchange, int elem_type, int count, const void *const *a,
                                          const void *const *b, void *const *out, int64_t rows, int64_t cols,
                                          int64_t b_row_stride, void *cuda_stream, char *err_buf, size_t err_len);
/* The same exchange for ANY compiled row-reduction group: afirt_executor_launch_device with one more argument.
 * The descriptor's tiling dims describe this rank's column slice (contiguous arguments, as always on that
 * path); the kernel sends the slice's partial row sums through the exchange and writes the sums over all ranks
 * to the output.  Refused for other kernel classes.  Collective like the call above, and counted in the same
 * sequence of calls of the exchange; the executor and the exchange must be on the same device. */
int afirt_executor_launch_device_exchange(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                          const char *function_name, int num_inputs, const void **input_ptrs,
                                          const size_t *input_bytes, int num_outputs, void **output_ptrs,
                                          const size_t *output_bytes, const uint8_t *tiling_data, size_t tiling_len,
                                          int block_dim, uint32_t magic, void *workspace, size_t workspace_bytes,
                                          void *cuda_stream, AfirtRowsumExchange exchange, char *err_buf, size_t err_len);
int afirt_rowsum_exchange_status(AfirtRowsumExchange exchange, char *err_buf, size_t err_len);
void afirt_rowsum_exchange_destroy(AfirtRowsumExchange exchange);

/* No counterpart in the reference (one device, one table).  A row-gather group whose TABLE is sharded by rows over
 * the GPUs of a node (a table larger than one GPU's memory): afirt_executor_launch_device with the table given as
 * num_shards device pointers, shard s holding rows [s * rows_per_shard, (s + 1) * rows_per_shard) with the table's
 * row length.  The pointers may be other GPUs' memory mapped into this process (afirt_peer_import below, or peer
 * access inside one process); the kernel reads remote rows with plain loads over NVLink, so no exchange step and
 * no library collective is involved.  input_ptrs[table input] is ignored but must not be NULL (pass the first
 * shard); input_bytes[table input] is the WHOLE table's size, as the descriptor's dims imply.  Indices, the other
 * operands and the output are this GPU's, as always.  Refused for other kernel classes and for column gathers. */
int afirt_executor_launch_device_sharded_table(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                               const char *function_name, int num_inputs, const void **input_ptrs,
                                               const size_t *input_bytes, int num_outputs, void **output_ptrs,
                                               const size_t *output_bytes, const uint8_t *tiling_data, size_t tiling_len,
                                               int block_dim, uint32_t magic, void *workspace, size_t workspace_bytes,
                                               void *cuda_stream, int num_shards, const void **shard_ptrs,
                                               int64_t rows_per_shard, char *err_buf, size_t err_len);

/* Device memory of one process made addressable from another process's GPU on the same node (CUDA IPC).
 *   export   writes AFIRT_PEER_HANDLE_BYTES bytes describing device_ptr, which may point INSIDE an allocation (a
 *            framework's sub-allocation of a larger block); the memory must come from cudaMalloc;
 *   import   maps it for device_id in the calling process and returns the pointer (inside the exporting process it
 *            returns the original pointer, enabling peer access when device_id is another GPU); importing
 *            several pointers of one allocation shares one mapping;
 *   release  drops one import; the mapping goes with the last one.  The exporter keeps the memory alive until
 *            every importer has released it. */
#define AFIRT_PEER_HANDLE_BYTES 96
int afirt_peer_export(const void *device_ptr, uint8_t *out_handle, char *err_buf, size_t err_len);
int afirt_peer_import(int device_id, const uint8_t *handle, void **out_ptr, char *err_buf, size_t err_len);
int afirt_peer_release(void *imported_ptr, char *err_buf, size_t err_len);

/* Library identification: "afir-b200 <version> sm_100a". */
const char *afirt_runtime_version(void);

#ifdef __cplusplus
}
#endif

#endif /* AFIR_CAPI_RUNTIME_CUDA_H */
