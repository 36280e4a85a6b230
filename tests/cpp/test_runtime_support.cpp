// Hand-rolled checks of the host runtime (no GPU): npy I/O, tiling packing, output comparator, task graph,
// run manifest, execution session with an injected driver.  Exit code = number of failed expectations,
// the convention of the reference's test/tools/runtime/test_runtime.cpp and test_taskgraph_runtime.cpp.
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <filesystem>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>

#include "common/json.h"
#include "execution/execution_session.h"
#include "execution/profile_retention.h"
#include "execution/run_manifest.h"
#include "front/shape_inference.h"
#include "kernels/matmul_plan.h"
#include "support/npy_io.h"
#include "support/tiling_schema.h"

using namespace afir;

static int g_pass = 0, g_fail = 0;
#define EXPECT(cond, what)                                                    \
  do {                                                                        \
    if (cond) ++g_pass;                                                       \
    else { ++g_fail; std::cerr << "FAIL: " << what << " (" << __LINE__ << ")\n"; } \
  } while (0)

static std::string g_dir;
static std::string path(const std::string &leaf) { return g_dir + "/" + leaf; }
static void writeText(const std::string &p, const std::string &text) { std::ofstream(p) << text; }

static void testNpy() {
  NDArray a;
  a.dtype = NpyDType::F16;
  a.shape = {2, 3};
  a.allocate();
  const uint16_t one = 0x3C00;
  for (int i = 0; i < 6; ++i) std::memcpy(a.bytes.data() + 2 * i, &one, 2);
  EXPECT(saveNpy(path("h.npy"), a).ok(), "save f16");
  NDArray b;
  EXPECT(loadNpy(path("h.npy"), b).ok(), "load f16");
  EXPECT(b.dtype == NpyDType::F16 && b.shape == a.shape && b.bytes == a.bytes, "f16 round trip keeps 0x3C00");
  std::ifstream f(path("h.npy"), std::ios::binary);
  std::string head(10, '\0');
  f.read(head.data(), 10);
  const unsigned hlen = static_cast<unsigned char>(head[8]) | (static_cast<unsigned char>(head[9]) << 8);
  EXPECT(head.compare(0, 6, "\x93NUMPY") == 0 && head[6] == 1 && head[7] == 0, "version 1.0 header");
  EXPECT((10 + hlen) % 64 == 0, "header padded to 64 bytes");

  NDArray s16;
  s16.dtype = NpyDType::INT16;
  s16.shape = {3};
  s16.allocate();
  const int16_t vals[3] = {-32768, -1, 32767};
  std::memcpy(s16.bytes.data(), vals, sizeof vals);
  EXPECT(saveNpy(path("s16.npy"), s16).ok(), "save i16");
  NDArray s16b;
  EXPECT(loadNpy(path("s16.npy"), s16b).ok() && s16b.dtype == NpyDType::INT16 && s16b.bytes == s16.bytes, "i16 round trip (<i2)");

  NDArray c;
  c.dtype = NpyDType::BF16;
  c.shape = {4};
  c.allocate();
  const uint16_t bone = 0x3F80;
  for (int i = 0; i < 4; ++i) std::memcpy(c.bytes.data() + 2 * i, &bone, 2);
  EXPECT(saveNpy(path("b.npy"), c).ok(), "save bf16");
  std::ifstream fb(path("b.npy"), std::ios::binary);
  std::string all((std::istreambuf_iterator<char>(fb)), std::istreambuf_iterator<char>());
  EXPECT(all.find("'descr': '<V2'") != std::string::npos, "bf16 stored as <V2");
  EXPECT(all.find("'shape': (4,)") != std::string::npos, "1-D shape keeps the trailing comma");
  NDArray d;
  EXPECT(loadNpy(path("b.npy"), d).ok() && d.dtype == NpyDType::BF16 && d.bytes == c.bytes, "bf16 round trip keeps 0x3F80");

  for (NpyDType t : {NpyDType::F32, NpyDType::INT8, NpyDType::INT32, NpyDType::INT64}) {
    NDArray x;
    x.dtype = t;
    x.shape = {3, 1, 2};
    x.allocate();
    for (size_t i = 0; i < x.bytes.size(); ++i) x.bytes[i] = static_cast<uint8_t>(i * 7 + 1);
    NDArray y;
    EXPECT(saveNpy(path("t.npy"), x).ok() && loadNpy(path("t.npy"), y).ok() && y.dtype == t && y.shape == x.shape && y.bytes == x.bytes,
           std::string("round trip ") + npyDTypeName(t));
  }
  // a column-major file (numpy writes one for the result of indexing columns with an index array) is brought into
  // row-major order: take a saved [2,3,4] i32 array, store its elements in column-major order, flip the header flag
  {
    NDArray x;
    x.dtype = NpyDType::INT32;
    x.shape = {2, 3, 4};
    x.allocate();
    for (int i = 0; i < 24; ++i) std::memcpy(x.bytes.data() + 4 * i, &i, 4);
    EXPECT(saveNpy(path("c_order.npy"), x).ok(), "save i32 [2,3,4]");
    std::ifstream in(path("c_order.npy"), std::ios::binary);
    std::string file((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
    const size_t flag = file.find("'fortran_order': False");
    EXPECT(flag != std::string::npos, "the header names the order");
    file.replace(flag, 22, "'fortran_order': True ");
    const size_t data = file.size() - 96;
    for (int i0 = 0; i0 < 2; ++i0)
      for (int i1 = 0; i1 < 3; ++i1)
        for (int i2 = 0; i2 < 4; ++i2) {
          const int value = (i0 * 3 + i1) * 4 + i2, at = i0 + 2 * (i1 + 3 * i2);
          std::memcpy(&file[data + 4 * at], &value, 4);
        }
    { std::ofstream(path("f_order.npy"), std::ios::binary) << file; }
    NDArray y;
    EXPECT(loadNpy(path("f_order.npy"), y).ok() && y.shape == x.shape && y.bytes == x.bytes, "column-major [2,3,4] loads in row-major order");
    // rank 1 and single elements have one order only
    NDArray v;
    v.dtype = NpyDType::F32;
    v.shape = {5};
    v.allocate();
    for (size_t i = 0; i < v.bytes.size(); ++i) v.bytes[i] = static_cast<uint8_t>(i);
    EXPECT(saveNpy(path("v.npy"), v).ok(), "save f32 [5]");
    std::ifstream vin(path("v.npy"), std::ios::binary);
    std::string vfile((std::istreambuf_iterator<char>(vin)), std::istreambuf_iterator<char>());
    vfile.replace(vfile.find("'fortran_order': False"), 22, "'fortran_order': True ");
    { std::ofstream(path("vf.npy"), std::ios::binary) << vfile; }
    NDArray w;
    EXPECT(loadNpy(path("vf.npy"), w).ok() && w.bytes == v.bytes, "rank 1 is the same in both orders");
  }
  NDArray e;
  EXPECT(loadNpy(path("missing.npy"), e).message().find("Cannot open:") == 0, "missing file message");
  writeText(path("junk.npy"), "not an npy file at all");
  EXPECT(loadNpy(path("junk.npy"), e).message().find("Not a .npy file:") == 0, "bad magic message");
  {
    std::string trunc = all.substr(0, all.size() - 3);
    std::ofstream(path("trunc.npy"), std::ios::binary) << trunc;
    EXPECT(loadNpy(path("trunc.npy"), e).message().find("Truncated data in:") == 0, "truncated data message");
  }
  {
    // a header that claims far more than the file holds is refused before anything of that size is allocated
    std::string huge = all;
    const size_t at = huge.find("'shape': (4,)");
    huge.replace(at, 13, "'shape': (99999999994, 6)");
    std::ofstream(path("huge.npy"), std::ios::binary) << huge;
    EXPECT(loadNpy(path("huge.npy"), e).message().find("Truncated data in:") == 0, "a claimed shape beyond the file's size");
    std::string wrap = all;
    wrap.replace(wrap.find("'shape': (4,)"), 13, "'shape': (4294967296, 4294967296, 4294967296)");
    std::ofstream(path("wrap.npy"), std::ios::binary) << wrap;
    EXPECT(loadNpy(path("wrap.npy"), e).message().find("Truncated data in:") == 0, "a shape whose byte count wraps around 64 bits");
  }
  {
    std::string f8 = all;
    f8.replace(f8.find("<V2"), 3, "<f8");
    std::ofstream(path("f8.npy"), std::ios::binary) << f8;
    EXPECT(loadNpy(path("f8.npy"), e).message().find("Unsupported dtype '<f8':") == 0, "unsupported dtype message");
  }
}

static void testTiling() {
  writeText(path("space.json"), R"({"kernel":"k","tiling_params":[{"name":"TB_M","type":"int64"},{"name":"B","type":"int32"},{"name":"dim_arg0_0"}]})");
  TilingSchema schema;
  EXPECT(TilingSchema::fromJsonFile(path("space.json"), schema).ok() && schema.fields().size() == 3, "schema loads");
  EXPECT(schema.fields()[2].type == "int64", "type defaults to int64");
  std::vector<uint8_t> bytes;
  EXPECT(schema.pack({{"TB_M", 16}, {"B", 2}, {"dim_arg0_0", 640}}, bytes).ok() && bytes.size() == 20, "int64 + int32 + int64 = 20 bytes");
  int64_t a, c;
  int32_t b;
  std::memcpy(&a, bytes.data(), 8);
  std::memcpy(&b, bytes.data() + 8, 4);
  std::memcpy(&c, bytes.data() + 12, 8);
  EXPECT(a == 16 && b == 2 && c == 640, "little-endian values in schema order");
  EXPECT(schema.pack({{"TB_M", 16}}, bytes).message().find("tiling param count mismatch: got 1, expected 3 (TB_M, B, dim_arg0_0)") == 0, "count mismatch");
  EXPECT(schema.pack({{"B", 1}, {"TB_M", 2}, {"dim_arg0_0", 3}}, bytes).message().find("tiling param name mismatch at position 0: got 'B', expected 'TB_M'") == 0,
         "name mismatch");
  TilingBinding tb;
  EXPECT(packTilingBytes(tb, bytes).ok() && bytes.empty(), "absent tiling packs to nothing");
  tb.present = true;
  tb.schemaPath = path("space.json");
  tb.params = "dim_arg0_0=640, B=2,TB_M=16";
  EXPECT(packTilingBytes(tb, bytes).ok() && bytes.size() == 20, "schema + named params in any order");
  tb.params = "TB_M=16,B=2";
  EXPECT(packTilingBytes(tb, bytes).message() == "tiling params missing field: dim_arg0_0", "missing named field");
  std::ofstream(path("tiling.bin"), std::ios::binary) << std::string("\x01\x02\x03\x04", 4);
  tb.binaryPath = path("tiling.bin");
  EXPECT(packTilingBytes(tb, bytes).ok() && bytes.size() == 4 && bytes[3] == 4, "binary file wins over schema");
  TilingBinding only;
  only.present = true;
  only.params = "A=1";
  EXPECT(packTilingBytes(only, bytes).message() == "tiling params require either a schema path or a binary path", "params alone are refused");
  TilingSchema bad;
  writeText(path("bad.json"), R"({"kernel":"k"})");
  EXPECT(TilingSchema::fromJsonFile(path("bad.json"), bad).message().find("missing 'tiling_params' array") != std::string::npos, "missing tiling_params");
}

static NDArray f32Array(std::vector<float> v) {
  NDArray a;
  a.dtype = NpyDType::F32;
  a.shape = {static_cast<int64_t>(v.size())};
  a.allocate();
  std::memcpy(a.bytes.data(), v.data(), v.size() * 4);
  return a;
}

static void testComparator() {
  OutputComparisonResult r;
  EXPECT(compareRuntimeOutputs({f32Array({1, 2, 3})}, {f32Array({1, 2, 3})}, 0.0, 0.0, r).ok() && r.passed && r.maxAbsDiff == 0.0, "exact match passes at zero tolerance");
  EXPECT(compareRuntimeOutputs({f32Array({1, 2, 3.5f})}, {f32Array({1, 2, 3})}, 0.1, 0.1, r).ok() && !r.passed, "mismatch fails");
  EXPECT(r.maxAbsDiff == 0.5 && r.errorMessage.find("output comparison failed: max_abs_diff=0.5") == 0, "reports max_abs_diff");
  EXPECT(compareRuntimeOutputs({f32Array({100.5f})}, {f32Array({100})}, 0.0, 1e-2, r).ok() && r.passed, "rtol scales with |expected|");
  EXPECT(compareRuntimeOutputs({f32Array({1})}, {}, 1, 1, r).message() == "output count mismatch: got 1, expected 0", "count mismatch is structural");
  EXPECT(compareRuntimeOutputs({f32Array({1, 2})}, {f32Array({1})}, 1, 1, r).message() == "output 0 shape mismatch", "shape mismatch");
  NDArray h = f32Array({1});
  h.dtype = NpyDType::INT32;
  EXPECT(compareRuntimeOutputs({h}, {f32Array({1})}, 1, 1, r).message() == "output 0 dtype mismatch", "dtype mismatch");
  NDArray half;
  half.dtype = NpyDType::F16;
  half.shape = {2};
  half.allocate();
  const uint16_t vals[2] = {0x3C00, 0x0001};
  std::memcpy(half.bytes.data(), vals, 4);
  EXPECT(elementAsFloat(half, 0) == 1.0f && elementAsFloat(half, 1) == 5.9604644775390625e-08f, "f16 widening incl. subnormals");
}

static RuntimeTask makeTask(const std::string &id, std::vector<std::string> deps = {}) {
  RuntimeTask t;
  t.taskId = id;
  t.dependencies = std::move(deps);
  t.artifact.kernelName = "k";
  return t;
}

static void testTaskGraph() {
  TaskGraph g;
  EXPECT(g.addTask(makeTask("")).message() == "empty task id", "empty id");
  EXPECT(g.addTask(makeTask("a")).ok() && g.addTask(makeTask("a")).message() == "duplicate task id", "duplicate id");
  EXPECT(g.addTask(makeTask("c", {"b"})).ok() && g.addTask(makeTask("b", {"a"})).ok(), "add out of order");
  std::vector<std::string> ids;
  EXPECT(g.topologicalOrder(ids).ok() && ids == std::vector<std::string>({"a", "b", "c"}), "dependency order");
  TaskGraph unknown;
  unknown.addTask(makeTask("x", {"nope"}));
  EXPECT(unknown.topologicalOrder(ids).message() == "unknown task dependency", "unknown dependency");
  TaskGraph cyc;
  cyc.addTask(makeTask("p", {"q"}));
  cyc.addTask(makeTask("q", {"p"}));
  EXPECT(cyc.topologicalOrder(ids).message() == "task graph contains a cycle", "cycle");
}

class RecordingDriver final : public ExecutionBackendDriver {
public:
  std::vector<std::string> order;
  std::vector<std::string> seenInputs;
  std::string failOn;
  Status run(const ExecutionRequest &request, ExecutionResult &result) override {
    order.push_back(request.task.taskId);
    for (const auto &b : request.task.invocation.inputs) seenInputs.push_back(b.path);
    result.taskId = request.task.taskId;
    if (request.task.taskId == failOn) return Status::error("[cuda:kernel_launch] injected failure");
    return Status::success();
  }
};

static void testManifestAndSession() {
  ::mkdir(path("art").c_str(), 0755);
  writeText(path("art/k.bin"), "{}");
  writeText(path("art/manifest.txt"), "kernel_name=k\nsoc_version=sm_100a\nkernel_kind=vec\ndevice_binary_path=" + path("art/k.bin") + "\nmanifest_path=x\n");
  writeText(path("m.json"), std::string(R"({"backend":"cuda","artifact_root":")") + path("art") + R"(","tasks":[
    {"task_id":"second","dependencies":["first"],"inputs":[{"name":"x","source":"task_output","upstream_task":"first","upstream_output":"y"}],
     "outputs":[{"name":"z","shape":[4],"dtype":"f32"}],"block_dim":7,"atol":0.5,"rtol":0.25,"profiling":true,
     "tiling":{"schema":"s.json","params":"A=1"}},
    {"task_id":"first","inputs":[{"name":"in","path":"in.npy"}],"outputs":[{"name":"y","path":")" + path("y.npy") + R"(","shape":[2,2],"dtype":"bf16"}]}
  ]})");
  RunManifestSpec spec;
  EXPECT(loadRunManifest(path("m.json"), spec).ok() && spec.tasks.size() == 2, "manifest with tasks[] loads");
  const RuntimeTask &second = spec.tasks[0];
  EXPECT(second.invocation.blockDim == 7 && second.invocation.atol == 0.5 && second.invocation.rtol == 0.25 && second.invocation.enableProfiling, "scalar fields");
  EXPECT(second.invocation.inputs[0].sourceKind == BindingSourceKind::TaskOutput && second.invocation.inputs[0].upstreamOutputName == "y", "task_output binding");
  EXPECT(second.invocation.tiling.present && second.invocation.tiling.params == "A=1", "tiling binding");
  EXPECT(spec.tasks[1].invocation.outputs[0].dtype.value() == NpyDType::BF16 && spec.tasks[1].invocation.outputs[0].shape->size() == 2, "shape and dtype");
  EXPECT(spec.tasks[1].invocation.atol == 1.0 && spec.tasks[1].invocation.rtol == 1e-2 && spec.tasks[1].invocation.workspaceSize == 8192, "reference defaults");
  TaskGraph graph;
  EXPECT(buildTaskGraph(spec, graph).ok(), "artifact roots resolve");

  auto driver = std::make_shared<RecordingDriver>();
  ExecutionSession session("cuda", driver);
  SessionPlan plan;
  EXPECT(session.plan(graph, plan).ok() && plan.orderedTaskIds == std::vector<std::string>({"first", "second"}), "plan is dependency ordered");
  SessionRunSummary summary = session.run(graph, path("work"));
  EXPECT(summary.success && driver->order == std::vector<std::string>({"first", "second"}), "runs in order");
  EXPECT(driver->seenInputs.size() == 2 && driver->seenInputs[1] == path("y.npy"), "upstream output resolves to the producer's file");
  EXPECT(summary.profileTrace.counters["planned_task_count"] == 2 && summary.profileTrace.counters["serialized_launch_count"] == 2, "counters");

  auto failing = std::make_shared<RecordingDriver>();
  failing->failOn = "first";
  ExecutionSession s2("cuda", failing);
  summary = s2.run(graph, path("work2"));
  EXPECT(!summary.success && failing->order.size() == 1, "first failure stops the session");
  EXPECT(summary.errorStage == "kernel_launch" && summary.errorMessage == "injected failure", "stage tag parsed out of the message");

  RunManifestSpec badSpec;
  writeText(path("bad1.json"), R"({"artifact_root":"x","task_id":"t"})");
  EXPECT(loadRunManifest(path("bad1.json"), badSpec).message() == "missing required string field: backend", "backend is required");
  writeText(path("bad2.json"), R"({"backend":"tpu","artifact_root":"x","task_id":"t"})");
  EXPECT(loadRunManifest(path("bad2.json"), badSpec).message() == "unsupported backend: tpu", "unknown backend");
  writeText(path("bad3.json"), R"({"backend":"cuda","task_id":"t"})");
  EXPECT(loadRunManifest(path("bad3.json"), badSpec).message() == "missing required string field: artifact_root", "artifact_root is required");
  writeText(path("bad4.json"), "{nope");
  EXPECT(loadRunManifest(path("bad4.json"), badSpec).message().find("invalid JSON in run manifest:") == 0, "invalid JSON");
  writeText(path("ok5.json"), std::string(R"({"backend":"sim","artifact_root":")") + path("art") + R"(","task_id":"solo"})");
  EXPECT(loadRunManifest(path("ok5.json"), badSpec).ok() && badSpec.tasks.size() == 1 && badSpec.backendName == "sim", "single-task form; reference backend names accepted");
  auto parts = parseErrorStage("[cuda:validate] output comparison failed");
  EXPECT(parts.first == "validate" && parts.second == "output comparison failed", "parseErrorStage");
  EXPECT(parseErrorStage("plain").first.empty(), "untagged message");
}

static void testProfileRetention() {
  // two artifacts, one with its score on the event, one whose score is read back from the file
  writeText(path("a.trace.json"), "{\"score\": 12.5, \"cycle_count\": 12.5}");
  writeText(path("b.trace.json"), "{\"cycle_count\": 4}");
  ProfileTrace trace;
  trace.sessionId = "sess-1";
  trace.attributes["scheduler_mode"] = "serial";
  trace.counters["planned_task_count"] = 2;
  trace.events.push_back({"a", "cuda", path("a.trace.json"), 12.5});
  trace.events.push_back({"b", "cuda", path("b.trace.json"), 0.0});
  RetainedProfileArtifacts kept;
  const std::string root = path("retained");
  EXPECT(retainProfileArtifacts(trace, root, kept).ok(), "retain two artifacts");
  EXPECT(kept.summaryPath == root + "/sess-1/session_summary.json", "summary path");
  EXPECT(kept.trace.events[0].artifactPath == root + "/sess-1/tasks/a.json" && kept.trace.events[1].artifactPath == root + "/sess-1/tasks/b.json",
         "events point at the retained copies");
  std::ifstream is(kept.summaryPath);
  std::string text((std::istreambuf_iterator<char>(is)), std::istreambuf_iterator<char>());
  json::Value summary;
  std::string err;
  EXPECT(json::parse(text, summary, err) && summary.isObject(), "summary is json");
  EXPECT(summary.getInt("task_count", 0) == 2 && summary.getInt("failed_task_count", -1) == 0, "task counts");
  EXPECT(summary.getDouble("total_score", 0) == 16.5 && summary.getDouble("total_cycle_count", 0) == 16.5, "score falls back to cycle_count");
  EXPECT(summary.getString("session_id") == "sess-1" && summary.getString("backend") == "cuda", "session id and backend");

  ProfileTrace missing = trace;
  missing.events[0].artifactPath = path("nope.json");
  Status s = retainProfileArtifacts(missing, root, kept);
  EXPECT(!s.ok() && s.message().find("cannot retain profile artifact") == 0, "missing artifact is an error");
  writeText(path("c.trace.json"), "[1, 2]");
  ProfileTrace bad = trace;
  bad.events = {{"c", "cuda", path("c.trace.json"), 0.0}};
  s = retainProfileArtifacts(bad, root, kept);
  EXPECT(!s.ok() && s.message().find("must be a json object") != std::string::npos, "non-object artifact is an error");

  // pruning: newest directories stay, plain files are not touched, a missing root is fine
  const std::string pr = path("prune");
  for (int i = 0; i < 5; ++i) {
    const std::string d = pr + "/s" + std::to_string(i);
    std::filesystem::create_directories(d);
    std::filesystem::last_write_time(d, std::filesystem::file_time_type::clock::now() - std::chrono::hours(10 - i));
  }
  writeText(pr + "/note.txt", "keep me");
  EXPECT(pruneRetainedProfileDirectories(pr, 2).ok(), "prune");
  EXPECT(std::filesystem::exists(pr + "/s4") && std::filesystem::exists(pr + "/s3") && !std::filesystem::exists(pr + "/s2") &&
             !std::filesystem::exists(pr + "/s0") && std::filesystem::exists(pr + "/note.txt"),
         "the two newest directories and the file remain");
  EXPECT(pruneRetainedProfileDirectories(path("no-such-root"), 1).ok(), "missing root is not an error");
  EXPECT(pruneKeepCountForNewSession(20) == 19 && pruneKeepCountForNewSession(0) == 0, "room for the new session");
  EXPECT(prepareRetainedRootForNewSession(pr, 2).ok() && !std::filesystem::exists(pr + "/s3") && std::filesystem::exists(pr + "/s4"),
         "preparing for a new session leaves limit - 1 directories");
}

// The planner behaviours the reference pins in test/unittests/Runtime/NativeMatmulPlannerTest.cpp:25-100 (default
// plan, hints honoured, batches refused, the plan is what gets applied, a deterministic description), for the
// B200 kernel's choices.
static void testMatmulPlanner() {
  using namespace afir::kernels;
  MatmulProblem big;
  big.M = big.N = big.K = 8192;
  MatmulPlan plan;
  EXPECT(matmulPlannerSupports(big), "8192^3 is supported");
  EXPECT(buildMatmulPlan(big, MatmulHints(), 148, plan).empty(), "default plan builds");
  EXPECT(plan.variant == MatmulVariant::Rows256 && plan.tileM == 256 && plan.tileN == 256 && plan.tileK == 64, "enough 256-row tiles: 256x256x64");
  EXPECT(plan.stages == 3 && plan.tilesM == 32 && plan.tilesN == 32 && plan.kBlocks == 128, "tile counts and ring depth");
  EXPECT(plan.blockDim == 148 && plan.band == 16 && plan.traverse == MatmulTraverse::FirstM, "one persistent CTA per SM, M first in bands of 16");
  EXPECT(plan.operandRingBytes == 3u * 65536u && plan.tmemColumns == 512 && !plan.epilogueOverlapsMainloop, "3 x 64 KB stages, all of tensor memory");
  EXPECT(describeMatmulPlan(plan) == "planned_block_dim=148 variant=rows256 traverse=FIRSTM band=16 tile=256x256x64 stages=3 tiles=32x32 "
                                     "k_blocks=128 ring_bytes=196608 tmem_cols=512 overlap_epilogue=0",
         "description is stable: " + describeMatmulPlan(plan));
  MatmulPlan again;
  buildMatmulPlan(big, MatmulHints(), 148, again);
  EXPECT(describeMatmulPlan(again) == describeMatmulPlan(plan), "same problem, same description");

  MatmulProblem small;
  small.M = 1024; small.N = 2048; small.K = 320;
  EXPECT(buildMatmulPlan(small, MatmulHints(), 148, plan).empty(), "small plan builds");
  EXPECT(plan.variant == MatmulVariant::Rows128 && plan.stages == 4 && plan.epilogueOverlapsMainloop, "too few 256-row tiles: 128-row tiles, double-buffered accumulators");
  EXPECT(plan.tileN == 256 && plan.tilesM == 8 && plan.tilesN == 8 && plan.kBlocks == 5 && plan.blockDim == 64, "grid capped by the number of tiles");

  // The 8192^3 problem M-sharded over 2, 4 and 8 GPUs keeps the 256-row tiles (at M = 1024, 128 tiles in one wave beat
  // 256 tiles of 128 rows in two: measured 101 us against 112 us).  At M = 4096 the 512 tiles are 4 waves over 148 SMs
  // but 7 rounds over 74 CTA pairs, each a little over half as long: the pair is chosen there (measured 381 against 390 us).
  for (int gpus : {2, 4, 8}) {
    MatmulProblem shard = big;
    shard.M = 8192 / gpus;
    EXPECT(buildMatmulPlan(shard, MatmulHints(), 148, plan).empty(), "shard plan builds");
    EXPECT(plan.variant == (gpus == 2 ? MatmulVariant::CtaPair : MatmulVariant::Rows256) && plan.tileN == 256 && plan.tilesN == 32 &&
               plan.tilesM == 32 / gpus,
           "M = 8192 / " + std::to_string(gpus) + ": 256 x 256 tiles, " + describeMatmulPlan(plan));
  }
  {
    MatmulProblem half = big;
    half.M = 4096;
    half.transposeB = true;  // B as [N, K]: the pair cannot split those tiles
    EXPECT(buildMatmulPlan(half, MatmulHints(), 148, plan).empty() && plan.variant == MatmulVariant::Rows256, "no pair for B as [N, K]");
    MatmulHints grid;
    grid.blockDim = 100;     // a grid asked for by the caller keeps the one-CTA-per-tile kernel
    half.transposeB = false;
    EXPECT(buildMatmulPlan(half, grid, 148, plan).empty() && plan.variant == MatmulVariant::Rows256, "no pair under a grid hint");
  }
  // a narrower tile is a hint: 148 tiles of 256 x 224 fill 148 SMs in whole waves
  MatmulHints width;
  width.tileN = 224;
  MatmulProblem eighth = big;
  eighth.M = 1024;
  EXPECT(buildMatmulPlan(eighth, width, 148, plan).empty() && plan.tileN == 224 && plan.tilesN == 37 && plan.blockDim == 148, "a tile-width hint is honoured");
  width.tileN = 192;
  EXPECT(buildMatmulPlan(big, width, 148, plan).empty() && plan.tileN == 192 && plan.tilesN == 43, "another width");
  width.tileN = 100;
  EXPECT(!buildMatmulPlan(big, width, 148, plan).empty(), "a tile width the kernel does not have is refused");

  MatmulHints hints;
  hints.variant = 3; hints.blockDim = 40; hints.band = 4;
  EXPECT(buildMatmulPlan(big, hints, 148, plan).empty(), "hinted plan builds");
  EXPECT(plan.variant == MatmulVariant::CtaPair && plan.blockDim == 40 && plan.band == 4 && plan.stages == 6, "hints are honoured");
  hints.blockDim = 41;
  buildMatmulPlan(big, hints, 148, plan);
  EXPECT(plan.blockDim == 40, "a CTA pair grid is even");
  big.transposeB = true;
  buildMatmulPlan(big, hints, 148, plan);
  EXPECT(plan.variant == MatmulVariant::Rows256, "B as [N, K] does not take the CTA pair");
  big.transposeB = false;

  MatmulProblem batched = big;
  batched.batchShape = {4};
  EXPECT(!matmulPlannerSupports(batched), "batched problems are unsupported");
  EXPECT(buildMatmulPlan(batched, MatmulHints(), 148, plan).find("batched") != std::string::npos, "and refused with a reason");
  MatmulProblem empty;
  EXPECT(!buildMatmulPlan(empty, MatmulHints(), 148, plan).empty(), "zero extents are refused");
  hints = MatmulHints();
  hints.variant = 7;
  EXPECT(!buildMatmulPlan(big, hints, 148, plan).empty(), "an unknown variant hint is refused");
}

// The shape rules of --afir-shape-inference (reference: lib/Dialect/AFIR/Ops/Basic/math.cpp:275-312 for the broadcast,
// include/Utils/AFIRShapeInferUtils.h:80-125 for the join with the declared result type).
static void testShapeInference() {
  using front::inferBroadcastShape;
  using front::joinShapes;
  using Shape = std::vector<int64_t>;
  Shape out;
  EXPECT(inferBroadcastShape({{4, 1, 31}, {1, 30, 1}}, out) && out == Shape({4, 30, 31}), "the reference's lit case");
  EXPECT(inferBroadcastShape({{8, -1}, {16}}, out) && out == Shape({8, 16}), "a later static extent replaces a dynamic one");
  EXPECT(inferBroadcastShape({{16}, {8, -1}}, out) && out == Shape({8, 16}), "a later dynamic extent changes nothing");
  EXPECT(inferBroadcastShape({{-1, 4}, {-1, 1}}, out) && out == Shape({-1, 4}), "unknown stays unknown");
  EXPECT(inferBroadcastShape({{1, 1}, {1}}, out) && out == Shape({1, 1}), "all ones");
  EXPECT(inferBroadcastShape({{}, {3}}, out) && out == Shape({3}), "rank 0 with rank 1");
  EXPECT(inferBroadcastShape({{5, 7}}, out) && out == Shape({5, 7}), "one operand");
  EXPECT(!inferBroadcastShape({{8, 4}, {8, 5}}, out), "static extents that differ do not broadcast");
  EXPECT(!inferBroadcastShape({{2, 3}, {4, 1, 3}, {5, 3}}, out), "a conflict in a middle position of three operands");
  EXPECT(joinShapes({-1, -1}, {8, 16}, out) && out == Shape({8, 16}), "a dynamic declaration takes the inference");
  EXPECT(joinShapes({8, -1}, {-1, 16}, out) && out == Shape({8, 16}), "each side fills the other's unknowns");
  EXPECT(joinShapes({8, 16}, {8, 16}, out) && out == Shape({8, 16}), "agreement");
  EXPECT(!joinShapes({8, 7}, {8, 4}, out), "a declared extent that contradicts the inference");
  EXPECT(!joinShapes({8}, {8, 4}, out), "ranks that differ");

  using front::inferConcatShape;
  EXPECT(inferConcatShape({{2, 4}, {3, 4}, {4, 4}}, 0, out) && out == Shape({9, 4}), "the reference's concat lit case");
  EXPECT(inferConcatShape({{4, 4}, {4, 4}}, 1, out) && out == Shape({4, 8}), "along the inner axis");
  EXPECT(inferConcatShape({{-1, 64}, {8, 64}}, 0, out) && out == Shape({-1, 64}), "a dynamic extent along the axis makes the sum dynamic");
  EXPECT(inferConcatShape({{8, 64}, {-1, 64}}, 0, out) && out == Shape({-1, 64}), "whatever the order");
  EXPECT(inferConcatShape({{8, -1}, {8, 64}}, 0, out) && out == Shape({16, -1}), "a dynamic extent elsewhere stays dynamic");
  EXPECT(!inferConcatShape({{8, 4}, {8, 5}}, 0, out), "parts that disagree off the axis");
  EXPECT(!inferConcatShape({{8, 4}, {8}}, 0, out), "ranks that differ");
  EXPECT(!inferConcatShape({{8, 4}}, 2, out) && !inferConcatShape({{8, 4}}, -1, out) && !inferConcatShape({}, 0, out), "axis outside the rank; no operand");

  using front::inferReducedShape;
  EXPECT(inferReducedShape({4, 5}, 0, out) && out == Shape({5}) && inferReducedShape({4, 5}, 1, out) && out == Shape({4}), "the reference's reduce lit case");
  EXPECT(inferReducedShape({2, -1, 8}, 2, out) && out == Shape({2, -1}), "dynamic extents pass through");
  EXPECT(!inferReducedShape({4, 5}, 2, out) && !inferReducedShape({4, 5}, -1, out) && !inferReducedShape({}, 0, out), "axis outside the rank");

  // the pass itself: text in, replacements out, a second run finds nothing
  front::Module m;
  const std::string text = "func.func @f(%a: tensor<2x1xf32>, %b: tensor<3xf32>) -> (tensor<?x?xf32>) {\n"
                           "  %0 = afir.add %a, %b : (tensor<2x1xf32>, tensor<3xf32>) -> tensor<?x?xf32>\n"
                           "  return %0 : tensor<?x?xf32>\n}\n";
  EXPECT(static_cast<bool>(front::parseModule(text, m)), "parse");
  int refined = 0;
  front::inferAfirShapes(m, &refined);
  const std::string printed = front::printModule(m);
  EXPECT(refined == 1 && m.replacements.size() == 3, "one op refined: op, return and function result rewritten");
  EXPECT(printed.find("-> tensor<2x3xf32> {") != std::string::npos && printed.find("return %0 : tensor<2x3xf32>\n}") != std::string::npos &&
             printed.find("(tensor<2x1xf32>, tensor<3xf32>) -> tensor<2x3xf32>\n") != std::string::npos,
         "printed module carries the refined types: " + printed);
  front::Module again;
  EXPECT(static_cast<bool>(front::parseModule(printed, again)), "the printed module parses");
  front::inferAfirShapes(again, &refined);
  EXPECT(refined == 0 && again.replacements.empty(), "idempotent");
}

int main() {
  char tmpl[] = "/tmp/afir-runtime-test-XXXXXX";
  if (!::mkdtemp(tmpl)) return 99;
  g_dir = tmpl;
  testNpy();
  testTiling();
  testComparator();
  testTaskGraph();
  testManifestAndSession();
  testProfileRetention();
  testMatmulPlanner();
  testShapeInference();
  std::cout << g_pass << " passed, " << g_fail << " failed\n";
  return g_fail;
}
