// Hand-rolled checks of task admission (no GPU): capacity accounting, session round robin, priority classes,
// admission quota, stream capacity, failure and release paths, counters, and the execution session running a
// graph through the scheduler on worker threads with an injected driver.  The behaviours are the ones the
// reference pins in test/tools/runtime/test_taskgraph_runtime.cpp:4676-5990 (resource scheduler, global
// scheduler, session-through-scheduler).  Exit code = number of failed expectations.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <iostream>
#include <limits>
#include <functional>
#include <set>
#include <thread>

#include "execution/execution_session.h"
#include "execution/global_scheduler.h"

using namespace afir;
using State = GlobalTaskRecord::State;

static int g_pass = 0, g_fail = 0;
#define EXPECT(cond, what)                                                    \
  do {                                                                        \
    if (cond) ++g_pass;                                                       \
    else { ++g_fail; std::cerr << "FAIL: " << what << " (" << __LINE__ << ")\n"; } \
  } while (0)

static RuntimeTask makeTask(const std::string &id, std::vector<std::string> deps = {}, size_t workspace = 16) {
  RuntimeTask t;
  t.taskId = id;
  t.dependencies = std::move(deps);
  t.invocation.workspaceSize = workspace;
  return t;
}
static TaskGraph makeGraph(std::initializer_list<RuntimeTask> tasks) {
  TaskGraph g;
  for (const RuntimeTask &t : tasks) g.addTask(t);
  return g;
}
static BackendCapabilities streamCaps(size_t tasks, size_t streams) {
  BackendCapabilities c;
  c.supportsConcurrentDispatch = true;
  c.supportsConcurrentExecution = true;
  c.maxConcurrentTasks = tasks;
  c.maxConcurrentStreams = streams;
  return c;
}
static std::string acquire(GlobalScheduler &s, const SessionHandle &h) {
  std::optional<RuntimeTask> t;
  bool drained = false;
  if (!s.tryAcquireTask(h.sessionId(), t, &drained).ok() || !t) return drained ? "<drained>" : "<none>";
  return t->taskId;
}

// ---------------------------------------------------------------------------------------------------
// ResourceScheduler
// ---------------------------------------------------------------------------------------------------

static void testReserveAndRelease() {
  ResourceScheduler rs;
  rs.configureSimDispatchLanes(1);
  rs.configureDeviceSlots(1);
  rs.configureWorkspaceBudget(1024);
  TaskResourceRequirement req;
  req.workspaceBytes = 512;
  req.requiresSerializedLaunch = true;
  auto a = rs.tryReserve("s0", "t0", req);
  EXPECT(a.has_value(), "first host reservation fits");
  auto b = rs.tryReserve("s1", "t1", req);
  EXPECT(!b && rs.lastBlockReason() == ResourceBlockReason::SerializedLaunch, "one lane: the second launch waits");
  rs.release(*a);
  EXPECT(rs.tryReserve("s1", "t1", req).has_value(), "lane comes back on release");

  ResourceScheduler ws;
  ws.configureWorkspaceBudget(100);
  TaskResourceRequirement big;
  big.workspaceBytes = 101;
  EXPECT(!ws.tryReserve("s", "t", big) && ws.lastBlockReason() == ResourceBlockReason::Workspace, "scratch over budget is refused");
  EXPECT(std::string(resourceBlockReasonName(ws.lastBlockReason())) == "workspace", "block reason has a name");
}

static void testForgedAndStaleReleases() {
  ResourceScheduler rs;
  rs.configureWorkspaceBudget(512);
  TaskResourceRequirement req;
  req.workspaceBytes = 512;
  auto live = rs.tryReserve("s0", "t0", req);
  EXPECT(live.has_value(), "reservation issued");
  ResourceReservation forged;  // same public fields, never issued
  forged.sessionId = live->sessionId;
  forged.taskId = live->taskId;
  forged.backendKind = live->backendKind;
  forged.workspaceBytes = live->workspaceBytes;
  rs.release(forged);
  EXPECT(!rs.tryReserve("s1", "t1", req), "a hand-built reservation releases nothing");
  rs.release(*live);
  EXPECT(rs.tryReserve("s1", "t1", req).has_value(), "the issued one does");

  ResourceScheduler twins;
  twins.configureWorkspaceBudget(1024);
  auto first = twins.tryReserve("s", "t", req);
  auto second = twins.tryReserve("s", "t", req);
  EXPECT(first && second, "two grants with identical public fields coexist");
  twins.release(*first);
  twins.release(*first);  // stale copy: must not free the twin
  EXPECT(twins.tryReserve("s", "t", req).has_value(), "one slot is free again");
  EXPECT(!twins.tryReserve("s", "t", req), "the twin still holds the other");
  EXPECT(twins.activeReservationCount() == 2, "two live grants");
}

static void testExclusiveDevice() {
  ResourceScheduler rs;
  rs.configureDeviceSlots(2);
  rs.configureWorkspaceBudget(1024);
  TaskResourceRequirement all;
  all.backendKind = ExecutionBackendKind::Cuda;
  all.workspaceBytes = 256;
  all.exclusiveDeviceAccess = true;
  auto whole = rs.tryReserve("s0", "t0", all);
  EXPECT(whole && whole->holdsDeviceSlot && rs.reservedDeviceSlots() == 2, "exclusive task takes every GPU");
  TaskResourceRequirement one;
  one.backendKind = ExecutionBackendKind::Cuda;
  one.workspaceBytes = 256;
  EXPECT(!rs.tryReserve("s1", "t1", one) && rs.lastBlockReason() == ResourceBlockReason::DeviceCapacity, "no GPU left beside it");
  rs.release(*whole);
  auto x = rs.tryReserve("s1", "t1", one), y = rs.tryReserve("s2", "t2", one);
  EXPECT(x && y, "two GPUs, two plain tasks");
  EXPECT(!rs.tryReserve("s3", "t3", one), "a third waits");
  EXPECT(!rs.tryReserve("s4", "t4", all), "exclusive needs all of them free");
  ResourceScheduler none;
  none.configureDeviceSlots(0);
  none.configureWorkspaceBudget(1024);
  EXPECT(!none.tryReserve("s", "t", all) && none.lastBlockReason() == ResourceBlockReason::DeviceCapacity, "no GPUs configured");
}

static void testStreams() {
  ResourceScheduler rs;
  rs.configureSimDispatchLanes(4);
  rs.configureDeviceSlots(4);
  rs.configureWorkspaceBudget(2048);
  rs.configureStreamCapacity(1);
  TaskResourceRequirement req;
  req.workspaceBytes = 16;
  req.requiresStream = true;
  req.streamUnits = 1;
  auto a = rs.tryReserve("s0", "t0", req);
  EXPECT(a && a->holdsStreamSlot && a->reservedStreamUnits == 1, "stream unit recorded on the reservation");
  EXPECT(!rs.tryReserve("s1", "t1", req) && rs.lastBlockReason() == ResourceBlockReason::StreamCapacity, "one stream: the second waits");
  EXPECT(rs.availableStreamCapacity() == 0 && rs.reservedStreamUnits() == 1, "stream counters");
  rs.release(*a);
  auto c = rs.tryReserve("s2", "t2", req);
  EXPECT(c.has_value(), "stream returns on release");

  TaskResourceRequirement alone;  // zero units + exclusive = one unit, nobody else
  alone.workspaceBytes = 16;
  alone.exclusiveStreamAccess = true;
  EXPECT(!rs.tryReserve("s3", "t3", alone) && rs.lastBlockReason() == ResourceBlockReason::ExclusiveStreamConflict,
         "exclusive request waits while a stream is out");
  rs.release(*c);
  auto e = rs.tryReserve("s4", "t4", alone);
  EXPECT(e && e->holdsStreamSlot && e->reservedStreamUnits == 1, "zero units normalise to one");
  EXPECT(!rs.tryReserve("s5", "t5", req) && rs.lastBlockReason() == ResourceBlockReason::ExclusiveStreamConflict,
         "shared request waits behind the exclusive holder");
  rs.release(*e);
  EXPECT(rs.tryReserve("s5", "t5", req).has_value(), "and runs after it");
}

static void testReconfigure() {
  ResourceScheduler rs;
  rs.configureWorkspaceBudget(1024);
  TaskResourceRequirement req;
  req.workspaceBytes = 512;
  auto a = rs.tryReserve("s0", "t0", req);
  rs.configureWorkspaceBudget(512);
  EXPECT(!rs.tryReserve("s1", "t1", req), "a lowered budget still counts what is out");
  rs.configureWorkspaceBudget(256);
  EXPECT(!rs.tryReserve("s1", "t1", TaskResourceRequirement()), "budget below what is out blocks even empty requests");
  rs.release(*a);
  rs.configureWorkspaceBudget(512);
  EXPECT(rs.tryReserve("s2", "t2", req).has_value(), "release restores the configured budget");
}

// ---------------------------------------------------------------------------------------------------
// GlobalScheduler
// ---------------------------------------------------------------------------------------------------

static void testSessionsAndErrors() {
  GlobalScheduler s;
  SessionHandle a, b, none;
  EXPECT(s.submit(ExecutionBackendKind::Host, makeGraph({makeTask("a0")}), a).ok(), "submit A");
  EXPECT(s.submit(ExecutionBackendKind::Host, makeGraph({makeTask("b0")}), b).ok(), "submit B");
  EXPECT(a.sessionId() != b.sessionId() && s.sessionCount() == 2, "two sessions, distinct ids");
  EXPECT(a.sessionId() == "global-session-0" && b.sessionId() == "global-session-1", "ids count up");
  Status empty = s.submit(ExecutionBackendKind::Host, TaskGraph(), none);
  EXPECT(!empty.ok() && empty.message() == "cannot submit empty task graph", "empty graph refused");
  TaskGraph cyc = makeGraph({makeTask("x", {"y"}), makeTask("y", {"x"})});
  EXPECT(!s.submit(ExecutionBackendKind::Host, cyc, none).ok(), "cyclic graph refused");

  std::optional<RuntimeTask> t;
  EXPECT(s.waitAndAcquireTask("nope", t).message() == "unknown global scheduler session: nope", "unknown session text");
  EXPECT(s.completeTask(a.sessionId(), "zz").message() == "unknown global scheduler task: global-session-0/zz", "unknown task text");
  EXPECT(s.completeTask(a.sessionId(), "a0").message() == "task is not running: global-session-0/a0", "complete before acquire refused");
  EXPECT(s.failTask(a.sessionId(), "a0").message() == "task is not running: global-session-0/a0", "fail before acquire refused");
  EXPECT(acquire(s, a) == "a0", "acquire a0");
  EXPECT(s.completeTask(a.sessionId(), "a0").ok(), "complete a0");
  EXPECT(acquire(s, a) == "<drained>", "session A drained");
  EXPECT(s.waitAndAcquireTask(a.sessionId(), t).ok() && !t, "blocking acquire returns empty on a drained session");
  s.releaseSession(a.sessionId());
  s.releaseSession(a.sessionId());  // twice is harmless
  EXPECT(s.sessionCount() == 1, "released session is gone");
}

static void testSingleLaneBlocksSecondSession() {
  GlobalScheduler s;
  s.configureResourceScheduler(1, 1, std::numeric_limits<size_t>::max(), 1);
  SessionHandle a, b;
  s.submit(ExecutionBackendKind::Host, makeGraph({makeTask("a0")}), a);
  s.submit(ExecutionBackendKind::Host, makeGraph({makeTask("b0")}), b);
  EXPECT(s.taskCountInState(State::Reserved) == 1 && s.taskCountInState(State::Ready) == 1, "one admitted, one waits");
  auto snap = s.observabilitySnapshot();
  EXPECT(snap.counters.at("scheduler.admission.resource_blocked") == 1, "the waiter is resource blocked");
}

static void testRoundRobin() {
  GlobalScheduler s;
  s.configureResourceScheduler(1, 1, 4096, 1);
  const BackendCapabilities caps = streamCaps(4, 1);
  SessionHandle a, b, c;
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("a0"), makeTask("a1")}), a);
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("b0")}), b);
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("c0")}), c);
  EXPECT(acquire(s, a) == "a0", "A goes first");
  EXPECT(acquire(s, b) == "<none>", "B has nothing reserved while A holds the stream");
  s.completeTask(a.sessionId(), "a0");
  EXPECT(acquire(s, a) == "<none>", "A does not get a second turn yet");
  EXPECT(acquire(s, b) == "b0", "B is next");
  s.completeTask(b.sessionId(), "b0");
  EXPECT(acquire(s, c) == "c0", "then C");
  s.completeTask(c.sessionId(), "c0");
  EXPECT(acquire(s, a) == "a1", "and A again");
  auto snap = s.observabilitySnapshot();
  EXPECT(snap.attributes.at("scheduler_policy") == "global_session_round_robin_baseline", "policy name");
  EXPECT(snap.attributes.at("scheduler_fairness_policy") == "session_round_robin", "fairness policy name");
  EXPECT(snap.counters.at("scheduler.fairness.session_order_size") == 3, "three sessions in the rotation");
  EXPECT(snap.counters.at("scheduler.fairness.starvation_prevented_total") >= 3, "turn changes are counted");
  EXPECT(snap.counters.at("scheduler.fairness.session_rotations_total") == 4, "four admissions");
}

static void testQuota() {
  GlobalScheduler s;
  s.configureResourceScheduler(2, 2, 4096, 2);
  const BackendCapabilities caps = streamCaps(4, 2);
  SessionSchedulingOptions one;
  one.maxAdmittedTasks = 1;
  SessionHandle a, b;
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("a0"), makeTask("a1")}), one, a);
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("b0")}), b);
  auto snap = s.observabilitySnapshot();
  EXPECT(snap.counters.at("scheduler.task.reserved") == 2, "quota leaves the second stream to B");
  EXPECT(snap.counters.at("scheduler.quota.blocked") == 1 && snap.counters.at("scheduler.quota.blocked_total") >= 1, "a1 waits on quota");
  EXPECT(acquire(s, a) == "a0" && acquire(s, b) == "b0", "both sessions run one task");
  EXPECT(acquire(s, a) == "<none>", "a1 not admitted while a0 holds the quota");
  s.completeTask(a.sessionId(), "a0");
  EXPECT(acquire(s, a) == "a1", "a1 admitted once a0 is done");
}

static void testPriority() {
  GlobalScheduler s;
  s.configureResourceScheduler(1, 1, 4096, 1);
  const BackendCapabilities caps = streamCaps(4, 1);
  SessionSchedulingOptions low, high;
  low.priorityClass = SessionPriorityClass::Low;
  high.priorityClass = SessionPriorityClass::High;
  SessionHandle l, n, h;
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("l0"), makeTask("l1")}), low, l);
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("n0")}), n);
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("h0"), makeTask("h1")}), high, h);
  EXPECT(acquire(s, l) == "l0", "first come holds the stream");
  auto snap = s.observabilitySnapshot();
  EXPECT(snap.counters.at("scheduler.priority.high_ready") == 1 && snap.counters.at("scheduler.priority.normal_ready") == 1 &&
             snap.counters.at("scheduler.priority.low_ready") == 1, "ready sessions per class");
  s.completeTask(l.sessionId(), "l0");
  EXPECT(acquire(s, h) == "h0", "high class first");
  s.completeTask(h.sessionId(), "h0");
  EXPECT(acquire(s, h) == "h1", "high class until it has nothing ready");
  s.completeTask(h.sessionId(), "h1");
  EXPECT(acquire(s, n) == "n0", "then normal");
  s.completeTask(n.sessionId(), "n0");
  EXPECT(acquire(s, l) == "l1", "then low");
}

static void testDefaultPolicy() {
  GlobalScheduler s;
  s.configureResourceScheduler(4, 4, 4096, 4);
  GlobalSchedulerPolicy policy;
  policy.defaultSessionScheduling.priorityClass = SessionPriorityClass::High;
  policy.defaultSessionScheduling.maxAdmittedTasks = 1;
  s.configurePolicy(policy);
  const BackendCapabilities caps = streamCaps(4, 4);
  SessionHandle byDefault, explicitOne;
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("d0"), makeTask("d1")}), byDefault);
  SessionSchedulingOptions free;  // normal priority, no quota
  s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("e0"), makeTask("e1")}), free, explicitOne);
  auto snap = s.observabilitySnapshot();
  EXPECT(snap.attributes.at("scheduler_default_priority_class") == "high", "default class published");
  EXPECT(snap.counters.at("scheduler.policy.default_max_admitted_tasks") == 1, "default quota published");
  EXPECT(snap.counters.at("scheduler.task.reserved") == 3, "default quota holds d1 back, explicit options ignore the default");
  EXPECT(snap.counters.at("scheduler.quota.blocked") == 1, "d1 waits on the default quota");
}

static void testBackfill() {
  {  // high class at its quota: lower class uses the spare stream
    GlobalScheduler s;
    s.configureResourceScheduler(2, 2, 4096, 2);
    const BackendCapabilities caps = streamCaps(4, 2);
    SessionSchedulingOptions highOne;
    highOne.priorityClass = SessionPriorityClass::High;
    highOne.maxAdmittedTasks = 1;
    SessionHandle h, l;
    s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("h0"), makeTask("h1")}), highOne, h);
    s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("l0")}), l);
    auto snap = s.observabilitySnapshot();
    EXPECT(snap.counters.at("scheduler.task.reserved") == 2, "low class backfills");
    EXPECT(snap.counters.at("scheduler.quota.blocked") == 1, "h1 waits on quota");
    EXPECT(snap.counters.at("scheduler.priority.high_ready") == 0, "a session at its quota is not counted as ready");
    EXPECT(acquire(s, h) == "h0" && acquire(s, l) == "l0", "one each");
  }
  {  // high class asks for more scratch than is free: lower class fits
    GlobalScheduler s;
    s.configureResourceScheduler(2, 2, 32, 2);
    const BackendCapabilities caps = streamCaps(4, 2);
    SessionSchedulingOptions high;
    high.priorityClass = SessionPriorityClass::High;
    SessionHandle h, l;
    s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("h0", {}, 64)}), high, h);
    s.submit(ExecutionBackendKind::Host, caps, makeGraph({makeTask("l0", {}, 16)}), l);
    EXPECT(acquire(s, h) == "<none>" && acquire(s, l) == "l0", "the task that fits runs, whatever its class");
    auto snap = s.observabilitySnapshot();
    EXPECT(snap.counters.at("scheduler.admission.resource_blocked") == 1, "h0 is resource blocked");
    EXPECT(snap.counters.at("scheduler.admission.stream_blocked") == 0, "not by streams");
    EXPECT(snap.counters.at("scheduler.fairness.session_skips_total") >= 1, "the skipped turn is counted");
  }
}

static void testStreamsFailureAndRelease() {
  GlobalScheduler s;
  s.configureResourceScheduler(4, 4, 4096, 1);
  const BackendCapabilities caps = streamCaps(2, 1);
  SessionHandle a, w;
  s.submit(ExecutionBackendKind::Cuda, caps, makeGraph({makeTask("main"), makeTask("after", {"main"})}), a);
  s.submit(ExecutionBackendKind::Cuda, caps, makeGraph({makeTask("waiting")}), w);
  auto snap = s.observabilitySnapshot();
  EXPECT(snap.counters.at("scheduler.stream.reserved") == 1 && snap.counters.at("scheduler.stream.capacity_total") == 1, "one stream, taken");
  EXPECT(snap.counters.at("scheduler.admission.stream_blocked") == 1 && snap.counters.at("scheduler.admission.stream_blocked_total") == 1,
         "the other session waits for a stream");
  EXPECT(snap.counters.at("scheduler.device.reserved") == 1, "a GPU task holds a device slot");
  EXPECT(acquire(s, a) == "main", "main runs");
  EXPECT(s.failTask(a.sessionId(), "main").ok(), "main fails");
  EXPECT(s.taskCountInState(State::Failed) == 1 && s.taskCountInState(State::Cancelled) == 1, "its dependent is cancelled");
  EXPECT(acquire(s, a) == "<drained>", "failed session is drained");
  s.releaseSession(a.sessionId());
  snap = s.observabilitySnapshot();
  EXPECT(snap.counters.at("scheduler.stream.reserved") == 1 && snap.counters.at("scheduler.stream.capacity_available") == 0 &&
             snap.counters.at("scheduler.task.reserved") == 1, "the freed stream goes straight to the waiting session");
  EXPECT(snap.counters.at("scheduler.transition.failed") == 1 && snap.counters.at("scheduler.transition.session_release") == 1, "transitions counted");
  EXPECT(acquire(s, w) == "waiting", "waiting runs");
  s.completeTask(w.sessionId(), "waiting");
  s.releaseSession(w.sessionId());
  snap = s.observabilitySnapshot();
  EXPECT(snap.counters.at("scheduler.stream.reserved") == 0 && snap.counters.at("scheduler.stream.capacity_available") == 1, "everything returned");
  EXPECT(snap.counters.at("scheduler.session_count") == 0 && snap.counters.at("scheduler.fairness.session_order_size") == 0, "no sessions left");
  EXPECT(snap.counters.at("scheduler.device.reserved") == 0 && snap.counters.at("scheduler.workspace.reserved_bytes") == 0, "no GPU or scratch held");
}

static void testDagAdvance() {
  GlobalScheduler s;
  SessionHandle h;
  TaskGraph g = makeGraph({makeTask("root"), makeTask("left", {"root"}), makeTask("right", {"root"}), makeTask("join", {"left", "right"})});
  s.submit(ExecutionBackendKind::Cuda, g, h);
  EXPECT(s.taskCountInState(State::Reserved) == 1 && s.taskCountInState(State::Submitted) == 3, "only the root is admitted");
  EXPECT(acquire(s, h) == "root", "root");
  size_t ready = 0;
  s.completeTask(h.sessionId(), "root", &ready);
  EXPECT(ready == 2 && s.taskCountInState(State::Reserved) == 2, "both children become ready and are admitted");
  EXPECT(acquire(s, h) == "left" && acquire(s, h) == "right", "children in id order");
  s.completeTask(h.sessionId(), "left", &ready);
  EXPECT(ready == 0 && acquire(s, h) == "<none>", "join waits for both");
  s.completeTask(h.sessionId(), "right", &ready);
  EXPECT(ready == 1 && acquire(s, h) == "join", "join after both");
  s.completeTask(h.sessionId(), "join");
  auto snap = s.observabilitySnapshot();
  EXPECT(snap.counters.at("scheduler.task.succeeded") == 4 && snap.counters.at("scheduler.transition.completed") == 4 &&
             snap.counters.at("scheduler.admission.reserved_total") == 4, "lifecycle counters");
  EXPECT(acquire(s, h) == "<drained>", "drained");
}

static void testBlockingAcquireWakesUp() {
  GlobalScheduler s;
  s.configureResourceScheduler(4, 4, 4096, 1);
  const BackendCapabilities caps = streamCaps(2, 1);
  SessionHandle a, b;
  s.submit(ExecutionBackendKind::Cuda, caps, makeGraph({makeTask("a0")}), a);
  s.submit(ExecutionBackendKind::Cuda, caps, makeGraph({makeTask("b0")}), b);
  std::string got;
  std::thread waiter([&] {
    std::optional<RuntimeTask> t;
    if (s.waitAndAcquireTask(b.sessionId(), t).ok() && t) got = t->taskId;
  });
  EXPECT(acquire(s, a) == "a0", "a0 holds the stream");
  std::this_thread::sleep_for(std::chrono::milliseconds(30));
  s.completeTask(a.sessionId(), "a0");  // frees the stream: the waiter must wake up with b0
  waiter.join();
  EXPECT(got == "b0", "blocked worker is woken when its task is admitted");
}

// ---------------------------------------------------------------------------------------------------
// ExecutionSession through the scheduler
// ---------------------------------------------------------------------------------------------------

namespace {
// Accepts tasks from several threads; "meet" tasks wait (bounded) until `meetCount` of them are inside run().
class FakeConcurrentDriver final : public ExecutionBackendDriver {
public:
  explicit FakeConcurrentDriver(size_t streams, int meetCount = 0) : streams_(streams), meetCount_(meetCount) {}
  BackendCapabilities capabilities() const override { return streamCaps(streams_, streams_); }
  ExecutionBackendKind kind() const override { return ExecutionBackendKind::Cuda; }
  Status run(const ExecutionRequest &request, ExecutionResult &result) override {
    result.taskId = request.task.taskId;
    std::unique_lock<std::mutex> lock(mutex_);
    order.push_back(request.task.taskId);
    for (const TensorBinding &in : request.task.invocation.inputs) seenInputPaths.insert(in.path);
    maxInside = std::max(maxInside, ++inside_);
    if (holdFirstUntil && order.size() == 1) {
      // the very first task stays inside the driver until the condition holds (5 s at most), so that what the
      // test wants to overlap with it really does, however fast the fake tasks are
      for (int i = 0; i < 1000 && !holdFirstUntil(); ++i) cv_.wait_for(lock, std::chrono::milliseconds(5));
    }
    if (request.task.taskId.rfind("meet", 0) == 0 && meetCount_ > 0) {
      ++met_;
      cv_.notify_all();
      cv_.wait_for(lock, std::chrono::seconds(2), [&] { return met_ >= meetCount_; });
    }
    --inside_;
    if (request.task.taskId.rfind("bad", 0) == 0) return Status::error("[cuda:kernel_launch] injected failure in " + request.task.taskId);
    result.profileTrace.counters["kernel_launches"] = 1;
    return Status::success();
  }
  std::vector<std::string> order;
  std::set<std::string> seenInputPaths;
  int maxInside = 0;
  std::function<bool()> holdFirstUntil;

private:
  size_t streams_;
  int meetCount_;
  int inside_ = 0, met_ = 0;
  std::mutex mutex_;
  std::condition_variable cv_;
};

RuntimeTask sessionTask(const std::string &id, std::vector<std::string> deps = {}) {
  RuntimeTask t = makeTask(id, std::move(deps));
  TensorBinding out;
  out.name = "out";
  t.invocation.outputs.push_back(out);
  for (const std::string &d : t.dependencies) {
    TensorBinding in;
    in.name = "from_" + d;
    in.sourceKind = BindingSourceKind::TaskOutput;
    in.upstreamTaskId = d;
    in.upstreamOutputName = "out";
    t.invocation.inputs.push_back(in);
  }
  return t;
}
} // namespace

static void testSessionRunsRootsConcurrently(const std::string &dir) {
  auto driver = std::make_shared<FakeConcurrentDriver>(4, 2);
  GlobalScheduler scheduler;
  ExecutionSession session("cuda", driver);
  session.setScheduler(&scheduler);
  TaskGraph g = makeGraph({sessionTask("meet0"), sessionTask("meet1"), sessionTask("join", {"meet0", "meet1"})});
  SessionRunSummary sum = session.run(g, dir + "/concurrent");
  EXPECT(sum.success, "concurrent session succeeds: " + sum.rawErrorMessage);
  EXPECT(driver->maxInside == 2, "both roots were inside the driver at the same time");
  EXPECT(driver->order.size() == 3 && driver->order.back() == "join", "join ran last");
  EXPECT(driver->seenInputPaths.count(dir + "/concurrent/meet0.out.npy") == 1 && driver->seenInputPaths.count(dir + "/concurrent/meet1.out.npy") == 1,
         "upstream outputs were bound as files of the session directory");
  const auto &tr = sum.profileTrace;
  EXPECT(tr.attributes.at("scheduler_mode") == "concurrent" && tr.attributes.at("scheduler_scope") == "global", "trace says concurrent");
  EXPECT(tr.attributes.at("scheduler_policy") == "global_session_round_robin_baseline", "scheduler attributes merged into the trace");
  EXPECT(tr.counters.at("max_in_flight_tasks") == 2 && tr.counters.at("planned_task_count") == 3, "in-flight and planned counters");
  EXPECT(tr.counters.at("scheduler.task.succeeded") == 3 && tr.counters.at("scheduler.stream.capacity_total") == 1024, "scheduler counters merged");
  EXPECT(tr.counters.at("frontier_count") == 2 && tr.counters.at("max_frontier_width") == 2, "frontiers: two roots, then the join");
  EXPECT(tr.counters.at("kernel_launches") == 3, "per-task counters are summed");
  EXPECT(sum.results.size() == 3 && sum.results[2].taskId == "join", "results come back in plan order");
  EXPECT(scheduler.sessionCount() == 0, "the session was released");
}

static void testSessionForcedSerial(const std::string &dir) {
  auto driver = std::make_shared<FakeConcurrentDriver>(4, 0);
  GlobalScheduler scheduler;
  ExecutionSession session("cuda", driver);
  session.setScheduler(&scheduler);
  ::setenv("ASCEND_RUNTIME_FORCE_SERIAL_SCHEDULER", "1", 1);
  SessionRunSummary sum = session.run(makeGraph({sessionTask("a"), sessionTask("b")}), dir + "/serial");
  ::unsetenv("ASCEND_RUNTIME_FORCE_SERIAL_SCHEDULER");
  EXPECT(sum.success && sum.profileTrace.attributes.at("scheduler_mode") == "serial", "environment switch forces the serial runner");
  EXPECT(driver->maxInside == 1 && sum.profileTrace.counters.at("serialized_launch_count") == 2, "one at a time");
  EXPECT(scheduler.observabilitySnapshot().counters.at("scheduler.admission.reserved_total") == 0, "scheduler untouched");
  // a single task never goes through the scheduler either
  sum = session.run(makeGraph({sessionTask("only")}), dir + "/single");
  EXPECT(sum.success && sum.profileTrace.attributes.at("scheduler_mode") == "serial", "single task runs serially");
}

static void testSessionFailureCancelsRest(const std::string &dir) {
  auto driver = std::make_shared<FakeConcurrentDriver>(2, 0);
  GlobalScheduler scheduler;
  ExecutionSession session("cuda", driver);
  session.setScheduler(&scheduler);
  TaskGraph g = makeGraph({sessionTask("bad0"), sessionTask("child", {"bad0"}), sessionTask("grandchild", {"child"})});
  SessionRunSummary sum = session.run(g, dir + "/failing");
  EXPECT(!sum.success && sum.errorStage == "kernel_launch" && sum.errorMessage == "injected failure in bad0", "first failure is reported with its stage");
  EXPECT(driver->order.size() == 1, "nothing downstream of the failure ran");
  EXPECT(sum.profileTrace.counters.at("scheduler.task.failed") == 1 && sum.profileTrace.counters.at("scheduler.task.cancelled") == 2, "dependents were cancelled");
  EXPECT(scheduler.sessionCount() == 0, "failed session was released");
}

static void testSessionsShareStreams(const std::string &dir) {
  // two sessions on one scheduler with a single stream: never more than one task inside the driver
  auto driver = std::make_shared<FakeConcurrentDriver>(4, 0);
  GlobalScheduler scheduler;
  scheduler.configureResourceScheduler(4, 1, 1 << 20, 1);
  // whichever session gets the stream first keeps it until the other one has submitted its graph too
  driver->holdFirstUntil = [&] { return scheduler.observabilitySnapshot().counters.at("scheduler.session_count") >= 2; };
  SessionRunSummary sums[2];
  std::thread threads[2];
  for (int i = 0; i < 2; ++i)
    threads[i] = std::thread([&, i] {
      ExecutionSession session("cuda", driver);
      session.setScheduler(&scheduler);
      const std::string p = i ? "y" : "x";
      sums[i] = session.run(makeGraph({sessionTask(p + "0"), sessionTask(p + "1"), sessionTask(p + "2")}), dir + "/shared" + p);
    });
  for (auto &t : threads) t.join();
  EXPECT(sums[0].success && sums[1].success, "both sessions finish");
  EXPECT(driver->maxInside == 1 && driver->order.size() == 6, "one stream on the node: tasks of both sessions take turns");
  EXPECT(scheduler.observabilitySnapshot().counters.at("scheduler.fairness.starvation_prevented_total") >= 1, "turns changed between the sessions");
}

int main() {
  char tmpl[] = "/tmp/afir-sched-XXXXXX";
  const char *d = ::mkdtemp(tmpl);
  const std::string dir = d ? d : "/tmp";
  testReserveAndRelease();
  testForgedAndStaleReleases();
  testExclusiveDevice();
  testStreams();
  testReconfigure();
  testSessionsAndErrors();
  testSingleLaneBlocksSecondSession();
  testRoundRobin();
  testQuota();
  testPriority();
  testDefaultPolicy();
  testBackfill();
  testStreamsFailureAndRelease();
  testDagAdvance();
  testBlockingAcquireWakesUp();
  testSessionRunsRootsConcurrently(dir);
  testSessionForcedSerial(dir);
  testSessionFailureCancelsRest(dir);
  testSessionsShareStreams(dir);
  std::cout << g_pass << " passed, " << g_fail << " failed\n";
  return g_fail;
}
