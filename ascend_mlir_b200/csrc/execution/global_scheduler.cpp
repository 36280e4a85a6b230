#include "execution/global_scheduler.h"

#include <algorithm>
#include <limits>

namespace afir {
namespace {

int rankOf(SessionPriorityClass p) { return p == SessionPriorityClass::High ? 2 : p == SessionPriorityClass::Low ? 0 : 1; }
const char *nameOf(SessionPriorityClass p) {
  return p == SessionPriorityClass::High ? "high" : p == SessionPriorityClass::Low ? "low" : "normal";
}
bool isStreamBlock(ResourceBlockReason r) {
  return r == ResourceBlockReason::StreamCapacity || r == ResourceBlockReason::ExclusiveStreamConflict;
}

} // namespace

GlobalScheduler &globalScheduler() {
  static GlobalScheduler scheduler;
  return scheduler;
}

size_t GlobalScheduler::Session::readyCount() const {
  size_t n = 0;
  for (const auto &t : tasks) n += t.second.state == State::Ready;
  return n;
}

BackendCapabilities GlobalScheduler::defaultCapabilitiesForBackend(ExecutionBackendKind backendKind) {
  BackendCapabilities caps;
  caps.supportsConcurrentDispatch = true;
  caps.maxConcurrentTasks = 1024;
  if (backendKind == ExecutionBackendKind::Host) {  // many tasks may queue, one launches at a time
    caps.supportsConcurrentExecution = false;
    caps.requiresSerializedLaunch = true;
    caps.maxConcurrentStreams = 1;
  } else {
    caps.supportsConcurrentExecution = true;
    caps.requiresSerializedLaunch = false;
    caps.maxConcurrentStreams = 1024;
  }
  return caps;
}

GlobalScheduler::GlobalScheduler() {
  // Effectively unlimited until the owner of the node configures real capacities.
  resources_.configureSimDispatchLanes(1024);
  resources_.configureDeviceSlots(1024);
  resources_.configureWorkspaceBudget(std::numeric_limits<size_t>::max());
  resources_.configureStreamCapacity(1024);
}

size_t GlobalScheduler::sessionCount() const {
  std::lock_guard<std::mutex> lock(mutex_);
  return sessions_.size();
}

void GlobalScheduler::configureResourceScheduler(size_t simDispatchLanes, size_t deviceSlots, size_t workspaceBudget,
                                                 size_t streamCapacity) {
  std::lock_guard<std::mutex> lock(mutex_);
  resources_.configureSimDispatchLanes(simDispatchLanes);
  resources_.configureDeviceSlots(deviceSlots);
  resources_.configureWorkspaceBudget(workspaceBudget);
  if (streamCapacity > 0) resources_.configureStreamCapacity(streamCapacity);
  admitLocked();
  changed_.notify_all();
}

void GlobalScheduler::configurePolicy(const GlobalSchedulerPolicy &policy) {
  std::lock_guard<std::mutex> lock(mutex_);
  policy_ = policy;
  changed_.notify_all();
}

size_t GlobalScheduler::countStateLocked(State state) const {
  size_t n = 0;
  for (const auto &s : sessions_)
    for (const auto &t : s.second.tasks) n += t.second.state == state;
  return n;
}

size_t GlobalScheduler::taskCountInState(State state) const {
  std::lock_guard<std::mutex> lock(mutex_);
  return countStateLocked(state);
}

// ---------------------------------------------------------------------------------------------------
// admission
// ---------------------------------------------------------------------------------------------------

void GlobalScheduler::markQuotaWaitLocked(Session &session) {
  for (auto &t : session.tasks) {
    TaskEntry &e = t.second;
    if (e.state != State::Ready || e.waitsForQuota) continue;
    e.waitsForQuota = true;
    ++totals_.quotaBlocked;
  }
}

GlobalScheduler::Attempt GlobalScheduler::admitOneLocked(const std::string &sessionId, Session &session) {
  if (session.failed) return Attempt::NothingReady;
  Attempt outcome = Attempt::NothingReady;
  for (auto &t : session.tasks) {
    TaskEntry &e = t.second;
    if (e.state != State::Ready) continue;
    if (session.quotaReached()) {
      markQuotaWaitLocked(session);
      return Attempt::QuotaBlocked;
    }
    e.waitsForQuota = false;
    std::optional<ResourceReservation> grant = resources_.tryReserve(sessionId, t.first, e.needs);
    if (!grant) {
      // remember why, count each task once per kind of wait, and look at the session's next ready task
      e.blockedBy = resources_.lastBlockReason();
      if (!e.waitsForResources) {
        e.waitsForResources = true;
        ++totals_.resourceBlocked;
      }
      if (!isStreamBlock(e.blockedBy)) {
        e.waitsForStreams = false;
      } else if (!e.waitsForStreams) {
        e.waitsForStreams = true;
        ++totals_.streamBlocked;
      }
      outcome = Attempt::ResourceBlocked;
      continue;
    }
    ++totals_.reserved;
    if (!lastAdmitted_.empty() && lastAdmitted_ != sessionId) ++totals_.turnsTaken;
    lastAdmitted_ = sessionId;
    ++session.admitted;
    e.clearWaits();
    e.reservation = std::move(grant);
    e.state = State::Reserved;
    return Attempt::Admitted;
  }
  return outcome;
}

void GlobalScheduler::admitLocked() {
  struct Candidate {
    size_t slot;
    int rank;
    Session *session;
  };
  while (!rotation_.empty()) {
    // One sweep over the sessions, starting behind the session that was admitted last.
    const size_t n = rotation_.size();
    std::vector<Candidate> sweep;
    int topRank = -1;
    for (size_t k = 0; k < n; ++k) {
      const size_t slot = (cursor_ + k) % n;
      auto it = sessions_.find(rotation_[slot]);
      if (it == sessions_.end() || it->second.failed) continue;
      Session &s = it->second;
      sweep.push_back({slot, rankOf(s.scheduling.priorityClass), &s});
      if (s.readyCount() == 0) continue;
      if (s.quotaReached()) {
        markQuotaWaitLocked(s);
        continue;
      }
      topRank = std::max(topRank, sweep.back().rank);
    }
    if (topRank < 0) return;
    // Highest class that can use what is free takes this sweep; every session of the class gets one try.
    bool admitted = false;
    for (int rank = topRank; rank >= 0 && !admitted; --rank) {
      for (const Candidate &c : sweep) {
        if (c.rank != rank) continue;
        const Attempt a = admitOneLocked(rotation_[c.slot], *c.session);
        if (a == Attempt::Admitted) {
          cursor_ = (c.slot + 1) % n;
          ++totals_.rotations;
          admitted = true;
        } else if (a != Attempt::NothingReady) {
          ++totals_.skips;
        }
      }
    }
    if (!admitted) return;
  }
}

void GlobalScheduler::giveBackLocked(Session &session, TaskEntry &entry) {
  if (!entry.reservation) return;
  resources_.release(*entry.reservation);
  entry.reservation.reset();
  if (session.admitted > 0) --session.admitted;
}

void GlobalScheduler::pointCursorAfterLocked(const std::string &sessionId) {
  auto it = std::find(rotation_.begin(), rotation_.end(), sessionId);
  if (it != rotation_.end()) cursor_ = (static_cast<size_t>(it - rotation_.begin()) + 1) % rotation_.size();
}

void GlobalScheduler::dropFromRotationLocked(const std::string &sessionId) {
  auto it = std::find(rotation_.begin(), rotation_.end(), sessionId);
  if (it != rotation_.end()) {
    const size_t slot = static_cast<size_t>(it - rotation_.begin());
    rotation_.erase(it);
    if (rotation_.empty()) cursor_ = 0;
    else {
      if (slot < cursor_) --cursor_;
      cursor_ %= rotation_.size();
    }
  }
  if (lastAdmitted_ == sessionId) lastAdmitted_.clear();
  else if (!lastAdmitted_.empty() && !rotation_.empty()) pointCursorAfterLocked(lastAdmitted_);
}

// ---------------------------------------------------------------------------------------------------
// sessions
// ---------------------------------------------------------------------------------------------------

Status GlobalScheduler::submit(ExecutionBackendKind kind, const TaskGraph &graph, SessionHandle &session) {
  return submit(kind, defaultCapabilitiesForBackend(kind), graph, policy_.defaultSessionScheduling, session);
}
Status GlobalScheduler::submit(ExecutionBackendKind kind, const TaskGraph &graph, const SessionSchedulingOptions &scheduling,
                               SessionHandle &session) {
  return submit(kind, defaultCapabilitiesForBackend(kind), graph, scheduling, session);
}
Status GlobalScheduler::submit(ExecutionBackendKind kind, const BackendCapabilities &caps, const TaskGraph &graph,
                               SessionHandle &session) {
  return submit(kind, caps, graph, policy_.defaultSessionScheduling, session);
}

Status GlobalScheduler::submit(ExecutionBackendKind kind, const BackendCapabilities &caps, const TaskGraph &graph,
                               const SessionSchedulingOptions &scheduling, SessionHandle &handle) {
  std::vector<RuntimeTask> order;
  if (Status s = graph.orderedTasks(order); !s) return s;
  if (order.empty()) return Status::error("cannot submit empty task graph");

  std::lock_guard<std::mutex> lock(mutex_);
  const std::string id = "global-session-" + std::to_string(nextOrdinal_++);
  Session &session = sessions_[id];
  session.backendKind = kind;
  session.scheduling = scheduling;
  rotation_.push_back(id);
  if (!lastAdmitted_.empty()) pointCursorAfterLocked(lastAdmitted_);

  for (const RuntimeTask &task : order) {
    TaskEntry &e = session.tasks[task.taskId];
    e.task = task;
    e.needs.backendKind = kind;
    e.needs.workspaceBytes = task.invocation.workspaceSize;
    e.needs.requiresSerializedLaunch = caps.requiresSerializedLaunch;
    // a GPU backend that cannot run two tasks side by side owns every device slot while it runs
    e.needs.exclusiveDeviceAccess =
        kind == ExecutionBackendKind::Cuda && (!caps.supportsConcurrentExecution || caps.maxConcurrentTasks <= 1);
    e.needs.requiresStream = caps.maxConcurrentStreams > 0;
    e.needs.streamUnits = e.needs.requiresStream ? 1 : 0;
    e.pendingDependencies = task.dependencies.size();
    e.state = task.dependencies.empty() ? State::Ready : State::Submitted;
  }
  for (const RuntimeTask &task : order)
    for (const std::string &dep : task.dependencies) session.tasks[dep].dependents.push_back(task.taskId);

  admitLocked();
  changed_.notify_all();
  handle = SessionHandle(id);
  return Status::success();
}

Status GlobalScheduler::tryAcquireTask(const std::string &sessionId, std::optional<RuntimeTask> &task, bool *drained) {
  std::lock_guard<std::mutex> lock(mutex_);
  task.reset();
  auto it = sessions_.find(sessionId);
  if (it == sessions_.end()) return Status::error("unknown global scheduler session: " + sessionId);
  for (auto &t : it->second.tasks) {
    if (t.second.state != State::Reserved) continue;
    t.second.state = State::Running;
    t.second.clearWaits();
    ++it->second.running;
    task = t.second.task;
    break;
  }
  if (drained) *drained = !task && it->second.drained();
  return Status::success();
}

Status GlobalScheduler::waitAndAcquireTask(const std::string &sessionId, std::optional<RuntimeTask> &task) {
  std::unique_lock<std::mutex> lock(mutex_);
  task.reset();
  while (true) {
    auto it = sessions_.find(sessionId);
    if (it == sessions_.end()) return Status::error("unknown global scheduler session: " + sessionId);
    for (auto &t : it->second.tasks) {
      if (t.second.state != State::Reserved) continue;
      t.second.state = State::Running;
      t.second.clearWaits();
      ++it->second.running;
      task = t.second.task;
      return Status::success();
    }
    if (it->second.drained()) return Status::success();
    changed_.wait(lock);
  }
}

Status GlobalScheduler::completeTask(const std::string &sessionId, const std::string &taskId, size_t *newlyReady) {
  std::lock_guard<std::mutex> lock(mutex_);
  if (newlyReady) *newlyReady = 0;
  auto sit = sessions_.find(sessionId);
  if (sit == sessions_.end()) return Status::error("unknown global scheduler session: " + sessionId);
  Session &session = sit->second;
  auto tit = session.tasks.find(taskId);
  if (tit == session.tasks.end()) return Status::error("unknown global scheduler task: " + sessionId + "/" + taskId);
  TaskEntry &e = tit->second;
  if (e.state != State::Running) return Status::error("task is not running: " + sessionId + "/" + taskId);

  giveBackLocked(session, e);
  e.clearWaits();
  e.state = State::Succeeded;
  ++totals_.completed;
  ++session.completed;
  if (session.running > 0) --session.running;
  if (!session.failed) {
    for (const std::string &next : e.dependents) {
      TaskEntry &d = session.tasks[next];
      if (d.state != State::Submitted || d.pendingDependencies == 0) continue;
      if (--d.pendingDependencies == 0) {
        d.state = State::Ready;
        d.clearWaits();
        if (newlyReady) ++*newlyReady;
      }
    }
  }
  admitLocked();
  changed_.notify_all();
  return Status::success();
}

Status GlobalScheduler::failTask(const std::string &sessionId, const std::string &taskId) {
  std::lock_guard<std::mutex> lock(mutex_);
  auto sit = sessions_.find(sessionId);
  if (sit == sessions_.end()) return Status::error("unknown global scheduler session: " + sessionId);
  Session &session = sit->second;
  auto tit = session.tasks.find(taskId);
  if (tit == session.tasks.end()) return Status::error("unknown global scheduler task: " + sessionId + "/" + taskId);
  TaskEntry &e = tit->second;
  if (e.state != State::Running) return Status::error("task is not running: " + sessionId + "/" + taskId);

  giveBackLocked(session, e);
  e.clearWaits();
  e.state = State::Failed;
  ++totals_.failed;
  session.failed = true;
  if (session.running > 0) --session.running;
  // everything of the session that has not started is cancelled; tasks already running finish on their own
  for (auto &t : session.tasks) {
    TaskEntry &other = t.second;
    if (other.state != State::Submitted && other.state != State::Ready && other.state != State::Reserved) continue;
    giveBackLocked(session, other);
    other.clearWaits();
    other.state = State::Cancelled;
  }
  admitLocked();  // what the session gave back may admit other sessions' tasks
  changed_.notify_all();
  return Status::success();
}

void GlobalScheduler::releaseSession(const std::string &sessionId) {
  std::lock_guard<std::mutex> lock(mutex_);
  auto sit = sessions_.find(sessionId);
  if (sit == sessions_.end()) return;
  for (auto &t : sit->second.tasks) giveBackLocked(sit->second, t.second);
  sessions_.erase(sit);
  ++totals_.sessionsReleased;
  dropFromRotationLocked(sessionId);
  admitLocked();
  changed_.notify_all();
}

// ---------------------------------------------------------------------------------------------------
// observability
// ---------------------------------------------------------------------------------------------------

SchedulerObservabilitySnapshot GlobalScheduler::observabilitySnapshot() const {
  std::lock_guard<std::mutex> lock(mutex_);
  SchedulerObservabilitySnapshot snap;
  auto &a = snap.attributes;
  auto &c = snap.counters;
  a["scheduler_policy"] = "global_session_round_robin_baseline";
  a["scheduler_fairness_policy"] = "session_round_robin";
  a["scheduler_priority_policy"] = "static_session_priority";
  a["scheduler_quota_policy"] = "session_admission_quota";
  a["scheduler_default_priority_class"] = nameOf(policy_.defaultSessionScheduling.priorityClass);
  a["resource_model_version"] = "v2";
  a["scheduler_stream_model"] = "enabled";

  c["scheduler.session_count"] = static_cast<int64_t>(sessions_.size());
  static const std::pair<const char *, State> kStates[] = {
      {"scheduler.task.submitted", State::Submitted}, {"scheduler.task.ready", State::Ready},
      {"scheduler.task.reserved", State::Reserved},   {"scheduler.task.running", State::Running},
      {"scheduler.task.succeeded", State::Succeeded}, {"scheduler.task.failed", State::Failed},
      {"scheduler.task.cancelled", State::Cancelled}};
  for (const auto &s : kStates) c[s.first] = static_cast<int64_t>(countStateLocked(s.second));

  int64_t waitingOnResources = 0, waitingOnStreams = 0, waitingOnQuota = 0;
  int64_t readyByRank[3] = {0, 0, 0};
  for (const auto &s : sessions_) {
    const Session &session = s.second;
    if (session.failed) continue;
    bool anyReady = false;
    for (const auto &t : session.tasks) {
      const TaskEntry &e = t.second;
      if (e.state != State::Ready) continue;
      anyReady = true;
      if (e.waitsForQuota) ++waitingOnQuota;
      if (e.waitsForResources && e.blockedBy != ResourceBlockReason::None) {
        ++waitingOnResources;
        if (isStreamBlock(e.blockedBy)) ++waitingOnStreams;
      }
    }
    if (anyReady && !session.quotaReached()) ++readyByRank[rankOf(session.scheduling.priorityClass)];
  }
  c["scheduler.admission.resource_blocked"] = waitingOnResources;
  c["scheduler.admission.resource_blocked_total"] = totals_.resourceBlocked;
  c["scheduler.stream.capacity_total"] = static_cast<int64_t>(resources_.configuredStreamCapacity());
  c["scheduler.stream.capacity_available"] = static_cast<int64_t>(resources_.availableStreamCapacity());
  c["scheduler.stream.reserved"] = static_cast<int64_t>(resources_.reservedStreamUnits());
  c["scheduler.admission.stream_blocked"] = waitingOnStreams;
  c["scheduler.admission.stream_blocked_total"] = totals_.streamBlocked;
  c["scheduler.quota.blocked"] = waitingOnQuota;
  c["scheduler.quota.blocked_total"] = totals_.quotaBlocked;
  c["scheduler.priority.high_ready"] = readyByRank[2];
  c["scheduler.priority.normal_ready"] = readyByRank[1];
  c["scheduler.priority.low_ready"] = readyByRank[0];
  c["scheduler.policy.default_max_admitted_tasks"] = static_cast<int64_t>(policy_.defaultSessionScheduling.maxAdmittedTasks);
  c["scheduler.admission.reserved_total"] = totals_.reserved;
  c["scheduler.transition.completed"] = totals_.completed;
  c["scheduler.transition.failed"] = totals_.failed;
  c["scheduler.transition.session_release"] = totals_.sessionsReleased;
  c["scheduler.fairness.cursor"] = static_cast<int64_t>(cursor_);
  c["scheduler.fairness.session_order_size"] = static_cast<int64_t>(rotation_.size());
  c["scheduler.fairness.session_rotations_total"] = totals_.rotations;
  c["scheduler.fairness.session_skips_total"] = totals_.skips;
  c["scheduler.fairness.starvation_prevented_total"] = totals_.turnsTaken;
  // re-hosted resources: GPUs and bytes of device scratch held by admitted tasks
  c["scheduler.device.reserved"] = static_cast<int64_t>(resources_.reservedDeviceSlots());
  c["scheduler.workspace.reserved_bytes"] = static_cast<int64_t>(
      std::min<size_t>(resources_.reservedWorkspaceBytes(), static_cast<size_t>(std::numeric_limits<int64_t>::max())));
  return snap;
}

} // namespace afir
