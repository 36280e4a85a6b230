// Launch descriptor: what `afir-translate -mlir-to-cuda` emits for one fused group and what the
// executor receives as the kernel "binary".  It names the kernel class in the prebuilt sm_100a
// library, the element type, the fused body and the TilingData layout (all-int64 fields: tile
// parameters first, then dim_arg<N>_<D> for every dynamic dimension, the reference's convention in
// lib/Conversion/AscendCPrepareForEmit/AscendCPrepareForEmitPass.cpp:200-216).
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "common/json.h"
#include "common/status.h"
#include "kernels/kernels.h"

namespace afir {

enum class DType { F32, F16, BF16, I32, I64, U8, I16 };
const char *dtypeName(DType t);
bool parseDType(const std::string &s, DType &out);
size_t dtypeBytes(DType t);

enum class KernelClass { Elementwise, RowReduce, Gather, Transpose, Matmul };
const char *kernelClassName(KernelClass c);

// A dimension: an integer literal or the name of a TilingData field.
struct DimExpr {
  bool literal = true;
  int64_t value = 0;
  std::string field;
};

// An affine view of one kernel argument over the group's iteration domain.
struct ViewSpec {
  int arg = -1;                 // kernel argument index: inputs first, then outputs
  DType dtype = DType::F32;
  std::vector<DimExpr> shape;   // shape of the whole argument tensor
  std::vector<int> map;         // per tensor dim: iteration dim it follows, or -1 for a fixed index
  std::vector<DimExpr> offset;  // per tensor dim: slice origin (extract_slice / concat offset)
};

struct GroupSpec {
  std::vector<DimExpr> domain;
  std::vector<ViewSpec> loads;
  ViewSpec store;
  kernels::BodyProgram body{};
  // gather groups: loads[0] is the table (map ignored), `indices` the index vector
  int gatherAxis = -1;
  ViewSpec indices;
};

struct MatmulSpec {
  int aArg = 0, bArg = 1, biasArg = -1, outArg = 3;
  DType inType = DType::BF16, outType = DType::BF16, biasType = DType::BF16;
  int epilogue = kernels::kEpiNone;
  double alpha = 0.0;
  DimExpr m, n, k;
  bool transposeB = false;  // B is [N, K]: out = A x B^T
};

struct TilingField {
  std::string name;
  int bytes = 8;  // int64 (8) or int32 (4), little-endian
};

struct LaunchDescriptor {
  std::string kernel;
  KernelClass kernelClass = KernelClass::Elementwise;
  DType dtype = DType::F32;
  int numInputs = 0, numOutputs = 0;
  std::vector<TilingField> tiling;
  std::vector<GroupSpec> groups;
  MatmulSpec matmul;
  // names of the tiling fields carrying B200 launch parameters (empty = library default)
  std::string ctaThreadsField, unrollField, splitColsField, stagesField, teamLanesField, bulkCopyField, streamStagesField, streamChunkField,
      warpRowsField, ctasPerSmField, tileKernelField, tileOrderField, variantField, streamRowsField, streamWarpsField;
  size_t tilingBytes() const;
};

// Container written by afirt_compiler_compile: "AFCU" | u32 version | u32 json length | json bytes, and from
// version 2 on the group's generated kernel: | u32 cubin length | cubin | u32 source length | CUDA source.
// Version 1 (descriptor only) is what matmul and bare-transpose groups get: they run on the library's own kernels.
constexpr uint32_t kContainerMagic = 0x55434641u;  // "AFCU" little-endian
constexpr uint32_t kContainerVersion = 1;
constexpr uint32_t kContainerVersionWithCode = 2;

// A kernel SOURCE file (what `afir-translate -mlir-to-cann` writes, the counterpart of the reference's
// step8_kernel.cpp) carries its launch descriptor in a leading comment block between these two marker lines, one
// line of JSON behind "// ".  embeddedDescriptorJson returns that JSON, or "" when the text holds no such block.
constexpr const char *kEmbeddedDescriptorBegin = "// afir-cuda-launch-descriptor-begin";
constexpr const char *kEmbeddedDescriptorEnd = "// afir-cuda-launch-descriptor-end";
std::string embeddedDescriptorJson(const std::string &sourceText);
std::string embedDescriptorComment(const std::string &compactJson);

Status parseDescriptorJson(const json::Value &root, LaunchDescriptor &out);
// Accepts the binary container or bare JSON text.
Status parseDescriptorBinary(const uint8_t *data, size_t len, LaunchDescriptor &out);
std::vector<uint8_t> wrapDescriptorContainer(const std::string &jsonText, const std::vector<uint8_t> &cubin = {},
                                             const std::string &source = std::string());
// The generated kernel inside a container (pointers into `data`; null / 0 where the container holds none).
struct ContainerCode {
  const uint8_t *cubin = nullptr;
  size_t cubinLen = 0;
  const char *source = nullptr;
  size_t sourceLen = 0;
};
ContainerCode containerCode(const uint8_t *data, size_t len);

// Decodes packed tiling bytes (schema order, little-endian) into named values.
Status unpackTiling(const LaunchDescriptor &d, const uint8_t *bytes, size_t len, std::map<std::string, int64_t> &out);

} // namespace afir
