// Host-visible launch interface of the sm_100a fused-group kernel library.
// Plain structs and pointers only: the runtime (.cpp, compiled by g++) fills these in from a
// launch descriptor plus TilingData values, the .cu files turn them into kernel launches.
#pragma once

#ifdef __CUDACC_RTC__
// Compiled at run time for a generated kernel (no host headers there): the fixed-width names this file uses.
typedef long long int64_t;
typedef unsigned long long uint64_t;
typedef unsigned long uintptr_t;
#else
#include <cstddef>
#include <cstdint>
#endif

typedef struct CUstream_st *cudaStream_t;

namespace afir {
namespace kernels {

enum ElemType : int { kF32 = 0, kF16 = 1, kBF16 = 2, kInt32 = 3, kInt16 = 4 };  // integers: elementwise groups only
enum IndexType : int { kI32 = 0, kI64 = 1 };

#ifndef __CUDACC_RTC__
inline int elemBytes(int t) { return (t == kF32 || t == kInt32) ? 4 : 2; }
#endif

// ---------------------------------------------------------------------------------------------
// Fused elementwise bodies.  A body is a short chain of arith ops over the values loaded from
// the group's views; every op rounds to the element type (no FMA contraction).
// ---------------------------------------------------------------------------------------------
enum BodyOpCode : int { kOpAdd = 0, kOpSub = 1, kOpMul = 2, kOpDiv = 3, kOpMax = 4, kOpMin = 5 };
enum BodySrcKind : int { kSrcView = 0, kSrcOp = 1, kSrcConst = 2 };

constexpr int kMaxViews = 6;   // loaded views per group (the gathered value counts as one)
constexpr int kMaxBodyOps = 8;

struct BodySrc {
  int kind;     // BodySrcKind
  int index;    // view index or op index
  float value;  // constant (already representable in the element type)
  int ivalue = 0;  // the same constant for integer element types, exact (a float holds integers up to 2^24 only)
};
struct BodyOp {
  int op;  // BodyOpCode
  BodySrc a, b;
};
struct BodyProgram {
  int numOps;  // 0 = identity of view 0
  BodyOp ops[kMaxBodyOps];
  // Filled by finishBodyProgram() for the interpreted kernels: how many views the ops read (highest index + 1)
  // and which op results some op other than the next one reads (those are the only ones kept in memory).
  int numViewsUsed = kMaxViews;
  unsigned int storeMask = 0xffffffffu;
};
#ifndef __CUDACC_RTC__
// Derives numViewsUsed and storeMask from the ops; a program left as parsed (all views, every result kept) is valid too.
void finishBodyProgram(BodyProgram &prog);
#endif

// Ids of the bodies compiled as straight-line specialisations (everything else runs through
// the op-by-op interpreter kernel, same results, lower throughput).
enum BodyId : int {
  kBodyInterpreted = -1,
  kBodyCopy = 0,          // v0
  kBodyAdd,               // v0 + v1
  kBodyMul,               // v0 * v1
  kBodyAddMulRhs,         // (v0 + v1) * v1
  kBodyAddMul,            // (v0 + v1) * v2
  kBodyMulAdd,            // v0 * v1 + v2
  kBodyReluAdd,           // max(v0, 0) + v1
  kBodyReluAddMul,        // (max(v0, 0) + v1) * v2
  kBodyRelu,              // max(v0, 0)
  kNumBodies
};

#ifndef __CUDACC_RTC__
// Returns the specialised body id computing `prog`, or kBodyInterpreted.
int matchBody(const BodyProgram &prog, int numViews);
#endif

// ---------------------------------------------------------------------------------------------
// Elementwise / broadcast / split / concat groups.
// Iteration domain collapsed to dims[0..2] (dims[2] innermost).  Each view is a device pointer
// (slice offsets already applied) with an element stride per domain dim; stride[2] is 1
// (contiguous, vector access) or 0 (broadcast along the inner dim, scalar access).
// ---------------------------------------------------------------------------------------------
struct ViewAccess {
  const void *base;
  int64_t stride[3];
};

struct ElementwiseLaunch {
  int elemType;
  int64_t dims[3];
  int numViews;
  ViewAccess views[kMaxViews];
  void *outBase;
  int64_t outStride[3];  // outStride[2] must be 1
  BodyProgram body;
  int ctaThreads;  // 0 = library default
  int unroll;      // vectors in flight per thread: 1, 2, 4 or 8; 0 = default
  int gridBlocks;  // 0 = library default
  int forceElementAccess = 0;  // 1: never use the block variant for transposed operands (testing, tuning)
  // One more (outermost) iteration dim above dims[0], for domains that keep four dims after collapsing
  // (out[b, h, s, d] = in[b, s, h, d]): extent and element strides per view and for the output.  Groups whose
  // views are all contiguous or constant along the inner dim take it as the grid's second dimension, one launch;
  // the others are launched once per index.
  int64_t outerCount = 1;
  int64_t viewOuterStride[kMaxViews] = {0, 0, 0, 0, 0, 0};
  int64_t outOuterStride = 0;
};
#ifndef __CUDACC_RTC__
// Returns a cudaError_t value (0 = success); *launched gets the number of kernels launched.
int launchElementwise(const ElementwiseLaunch &l, cudaStream_t stream, int *launched);
#endif

// ---------------------------------------------------------------------------------------------
// Row reduction: out[m] = sum_n body(views)(m, n), f32 accumulation from zero.
// dims = {rows, cols}; view strides are per (row, col) with the col stride 1 or 0.
// ---------------------------------------------------------------------------------------------
// Mailbox of a reduction whose reduced axis is sharded over GPUs (one process per GPU, or one process driving
// several).  Every pointer is a device address as seen from the launching GPU; peerSlots[p] / peerFlags[p] point
// into GPU p's mailbox (peer-mapped), at the place reserved for this rank.
constexpr int kMaxExchangeRanks = 8;
struct RowReduceExchange {
  // The mailbox has two halves used by alternate calls; the pointers below are those of half 0, the kernel adds
  // halfStride for odd call numbers.  The call number lives on the device (callWord), so that a launch carries
  // nothing that changes from call to call and a captured CUDA graph of such launches can be replayed.
  unsigned long long *peerEntries[kMaxExchangeRanks];  // where this rank's entries go on rank p: [rows] x {f32 sum, call number}
  const unsigned long long *myEntries;                 // local mailbox: [world, slotStride] entries, filled by all ranks
  unsigned int *doneCounter;                           // local: CTAs of the running launch that are done (plain kernel)
  unsigned int *status;                                // local: set to 1 when the wait for a rank ran out
  unsigned long long *callWord;                        // local: {completed calls : arrivals of the running launch}, 0 at creation
  int world;                                           // 0 = no exchange
  unsigned int epoch;                                  // device side only: the running call's number (filled in by the kernel)
  long long slotStride;                                // entries between two ranks' slots
  long long halfStride;                                // entries between the two halves
};

struct RowReduceLaunch {
  int elemType;
  int64_t rows, cols;
  int numViews;
  struct View2 { const void *base; int64_t rowStride; int64_t colStride; } views[kMaxViews];
  void *out;  // [rows], elemType
  BodyProgram body;
  int ctaThreads;   // 0 = default
  int teamLanes;    // threads cooperating on one row (power of two, 32..ctaThreads); 0 = choose
  int splitCols;    // column slices per row (>1 uses `workspace` for the partial sums); 0 = choose
  void *workspace;  // device scratch, at least rowReduceWorkspaceBytes(...) when splitCols > 1
  size_t workspaceBytes;
  int gridBlocks;
  int streamStages;      // staged variant: ring depth per warp (0 = default)
  int streamChunkBytes;  // staged variant: bytes per stage (0 = default)
  int forcePlainLoads;  // 1 = never use the bulk-copy staged variant (tuning / comparison)
  // Not null: the per-row sums are partial (this GPU holds a column slice).  The kernel stores them as f32 into
  // every rank's mailbox instead of `out`, waits (2 s at most) for the other ranks' partial sums and writes
  // out[m] = their sum in rank order.  Column slicing (splitCols) is not combined with it.
  const RowReduceExchange *exchange = nullptr;
  // Device word that the staged kernel sets to 1 when a wait for one of its copies runs out (the executor points
  // it into its own workspace, so concurrent executors do not read each other's time-outs); null = a word of the
  // library, one per device, read by rowReduceCheckStatus.
  unsigned int *status = nullptr;
};
#ifndef __CUDACC_RTC__
size_t rowReduceWorkspaceBytes(int64_t rows, int splitCols);
#endif
// How launchRowReduce runs a given reduction (see planRowReduce).
struct RowReducePlan {
  bool vector = false;        // 16-byte accesses (else one element at a time)
  int64_t vecPerRow = 0, vecPerSlice = 0;
  int slices = 1;             // column slices per row (> 1: partial sums through the workspace + a finalize kernel)
  int threads = 128, lanes = 32;
  int64_t grid = 1;
  int finalizeThreads = 256;
  int64_t finalizeGrid = 1;
  bool staged = false;        // the bulk-copy staged kernel: one streamed view through per-warp shared-memory rings
  int streamedView = -1, streamWarps = 0, streamStages = 0;
  unsigned int streamChunkBytes = 0;
  size_t smemBytes = 0;
};
#ifndef __CUDACC_RTC__
int planRowReduce(const RowReduceLaunch &l, int smCount, RowReducePlan &plan);
int chooseRowReduceSplit(int64_t rows, int64_t cols, int smCount);
int launchRowReduce(const RowReduceLaunch &l, cudaStream_t stream, int *launched);
// After the stream has been synchronised: non-zero when a staged-copy wait gave up.
int rowReduceCheckStatus(int device, char *errorText);
#endif

// ---------------------------------------------------------------------------------------------
// Gather + elementwise.  axis 0 (row gather, "embedding"): g(i,j) = table[idx[i], j];
// axis 1 (column gather, "index_select"): g(i,j) = table[i, idx[j]].  The gathered value is view 0
// of the body; views[1..] are ordinary (row, col) views.  Out-of-range indices leave the output
// element(s) untouched and raise *status (a device int64 counter) by one per bad index read.
// ---------------------------------------------------------------------------------------------
constexpr int kMaxTableShards = 8;
struct GatherLaunch {
  int elemType;
  int axis;
  int indexType;
  int64_t rows, cols;        // output shape
  const void *table;
  int64_t tableRows, tableCols, tableRowStride;
  const void *indices;
  int numViews;              // including the gathered value as view 0 (its ViewAccess is ignored)
  RowReduceLaunch::View2 views[kMaxViews];
  void *out;
  int64_t outRowStride;
  BodyProgram body;
  unsigned long long *status;  // device counter of out-of-range indices (may be null)
  int ctaThreads, unroll, gridBlocks;
  // row gather, bulk-copy staged kernel: opt-in (measured slower than the plain kernel on B200 for rows of
  // 256 bytes to 8 KB), used only when stagedCopies is set and the shapes qualify
  int stagedCopies = 0;
  int streamStages = 0;            // ring depth per warp, 2..8 (0 = 3)
  int streamRows = 0;              // rows per stage, 1..32 (0 = about 4 KB worth)
  int streamWarps = 0;             // warps per CTA, 1..16 (0 = 8)
  // Row gather from a table whose rows are split over several buffers (a table larger than one GPU's memory,
  // sharded over the GPUs of a node): shard s holds rows [s * rowsPerShard, (s + 1) * rowsPerShard) at
  // tableShards[s] with the same row stride; the pointers may be peer-mapped memory of other GPUs, read with plain
  // loads.  numShards = 0: the single `table` above.
  int numShards = 0;
  const void *tableShards[kMaxTableShards] = {nullptr};
  int64_t rowsPerShard = 0;
};
#ifndef __CUDACC_RTC__
int launchGather(const GatherLaunch &l, cudaStream_t stream, int *launched);
#endif

// ---------------------------------------------------------------------------------------------
// 2-D transpose out[c, r] = in[r, c] (2- or 4-byte elements): register-block kernel for 16-byte-aligned
// operands, padded shared-memory tile kernel otherwise.
// ---------------------------------------------------------------------------------------------
struct TransposeLaunch {
  int elemBytes;
  int64_t rows, cols;  // shape of `in`
  const void *in;
  int64_t inRowStride;
  void *out;
  int64_t outRowStride;
  int warpRows = 0;         // warps of a CTA stacked along the input rows: 1, 2, 4 or 8 (0 = default)
  int ctasPerSm = 0;        // persistent grid of SMs x this many CTAs (0 = one CTA per tile)
  int diagonalOrder = 0;    // tile order: 0 row-major (column-major when the input has few rows), 1 diagonal, 2 column-major
  int variant = 0;          // register blocks: 0 = whole lines stored (default), 1 = same with 2 blocks per thread, 2 = whole
                            // lines loaded, 3 = same, 2 blocks; 4 = the copy-engine kernel (16-bit elements; else as 0)
  int forceTileKernel = 0;  // 1: use the shared-memory tile kernel even when the operands are aligned
  unsigned int *status = nullptr;  // device word for wait time-outs of the copy-engine kernel, or null for the library's own
};
#ifndef __CUDACC_RTC__
int launchTranspose(const TransposeLaunch &l, cudaStream_t stream, int *launched);
// The copy-engine kernel (transpose_tma.cu): 16-bit elements, 16-byte-aligned operands and row strides.
bool transposeTmaApplies(const TransposeLaunch &l);
int launchTransposeTma(const TransposeLaunch &l, int smCount, cudaStream_t stream);
// 1 (and a message) when a wait of a launch without its own status word ran out since the last call; clears the word.
int transposeTmaCheckStatus(char *message, size_t messageBytes);
#endif

// ---------------------------------------------------------------------------------------------
// Matmul + bias + LeakyReLU:  out = epilogue(A[M,K] . B[K,N] + bias[N]); row-major, 16-bit inputs,
// f32 accumulation in tensor memory (tcgen05), operands staged by TMA.
// ---------------------------------------------------------------------------------------------
enum EpilogueKind : int { kEpiNone = 0, kEpiBiasAdd = 1, kEpiBiasAddLeakyRelu = 2, kEpiBiasAddRelu = 3 };

struct MatmulPlan;  // kernels/matmul_plan.h
struct MatmulLaunch {
  int inType;    // kF16 or kBF16 (A and B)
  int outType;   // kF32, kF16 or kBF16
  int biasType;  // kF32, kF16 or kBF16
  int64_t M, N, K;
  const void *A;  // [M,K] row-major
  const void *B;  // [K,N] row-major, or [N,K] row-major when bTransposed
  const void *bias;  // [N] or null
  void *out;      // [M,N] row-major
  int epilogue;
  float alpha;
  int gridBlocks;  // 0 = one persistent CTA per SM
  int stages;      // 0 = default
  int bTransposed = 0;  // 1: out = A x B^T with B stored [N,K] (no counterpart in the reference, whose matmul takes
                        // no transposes; it is how torch.nn.Linear keeps its weight)
  MatmulPlan *planOut = nullptr;  // receives the plan that was launched (variant, tile, grid, ...)
  // Device word that a kernel wait which runs out sets to (1 << 8) | role (the executor points it into its own
  // workspace); null = a word of the library, one per device, read by matmulCheckStatus.
  unsigned int *status = nullptr;
};
#ifndef __CUDACC_RTC__
// errorText (optional, >= 256 bytes) receives a description when the launch is refused or the
// kernel reports a bounded-wait timeout.
int launchMatmul(const MatmulLaunch &l, cudaStream_t stream, int *launched, char *errorText);
// After the stream has been synchronised: non-zero when a kernel wait gave up (see matmul_tcgen05.cu).
int matmulCheckStatus(int device, char *errorText);

// Library-wide helpers.
int deviceSmCount(int device);
const char *cudaErrorText(int code);

#endif

} // namespace kernels
} // namespace afir
