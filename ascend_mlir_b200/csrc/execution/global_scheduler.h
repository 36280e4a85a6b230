// Process-wide admission of task graphs ("sessions") onto the node's GPUs and streams.  Each submitted graph
// becomes a session; its tasks move Submitted -> Ready (dependencies done) -> Reserved (resources granted) ->
// Running (a worker took it) -> Succeeded | Failed | Cancelled.  Admission takes turns between sessions
// (round robin from a cursor that follows the last admitted session), serves higher priority classes first
// and falls back to lower ones when the higher ones cannot use the free resources, and stops admitting for
// a session that already holds its quota of admitted tasks.  The first failed task cancels everything of its
// session that has not started.  Workers block in waitAndAcquireTask() until a task of their session is
// reserved or the session has drained.
//
// Interface, state names, policy names, error texts and counter names follow the reference's
// include/Runtime/Execution/GlobalScheduler.h:23-159 and lib/Runtime/Execution/GlobalScheduler.cpp; the
// bookkeeping is per session here (ordered task table per session) instead of one table for all sessions.
#pragma once

#include <condition_variable>
#include <cstdint>
#include <map>
#include <mutex>
#include <optional>
#include <string>
#include <vector>

#include "common/status.h"
#include "execution/resource_scheduler.h"
#include "execution/task_graph.h"

namespace afir {

// What a backend tells the scheduler about itself (reference: include/Runtime/Execution/BackendCapabilities.h).
struct BackendCapabilities {
  bool supportsConcurrentDispatch = false;
  bool supportsConcurrentExecution = false;
  bool requiresSerializedLaunch = false;
  size_t maxConcurrentTasks = 1;
  size_t maxConcurrentStreams = 1;  // 0: the backend makes no statement about streams
};

enum class SessionPriorityClass { Low, Normal, High };

struct SessionSchedulingOptions {
  SessionPriorityClass priorityClass = SessionPriorityClass::Normal;
  size_t maxAdmittedTasks = 0;  // tasks of the session that may hold resources at once; 0 = no limit
};

struct GlobalSchedulerPolicy {
  SessionSchedulingOptions defaultSessionScheduling;
};

class SessionHandle {
public:
  SessionHandle() = default;
  explicit SessionHandle(std::string id) : id_(std::move(id)) {}
  const std::string &sessionId() const { return id_; }

private:
  std::string id_;
};

struct GlobalTaskRecord {
  enum class State { Submitted, Ready, Reserved, Running, Succeeded, Failed, Cancelled };
};

struct SchedulerObservabilitySnapshot {
  std::map<std::string, std::string> attributes;
  std::map<std::string, int64_t> counters;
};

class GlobalScheduler {
public:
  GlobalScheduler();

  Status submit(ExecutionBackendKind backendKind, const TaskGraph &graph, SessionHandle &session);
  Status submit(ExecutionBackendKind backendKind, const TaskGraph &graph, const SessionSchedulingOptions &scheduling,
                SessionHandle &session);
  Status submit(ExecutionBackendKind backendKind, const BackendCapabilities &capabilities, const TaskGraph &graph,
                SessionHandle &session);
  Status submit(ExecutionBackendKind backendKind, const BackendCapabilities &capabilities, const TaskGraph &graph,
                const SessionSchedulingOptions &scheduling, SessionHandle &session);

  // Blocks until a task of the session is reserved (returned, now Running) or the session is drained (empty).
  Status waitAndAcquireTask(const std::string &sessionId, std::optional<RuntimeTask> &task);
  // Non-blocking form of the above for single-threaded callers: `task` stays empty when nothing is reserved.
  Status tryAcquireTask(const std::string &sessionId, std::optional<RuntimeTask> &task, bool *drained = nullptr);
  Status completeTask(const std::string &sessionId, const std::string &taskId, size_t *newlyReady = nullptr);
  Status failTask(const std::string &sessionId, const std::string &taskId);
  void releaseSession(const std::string &sessionId);

  size_t sessionCount() const;
  void configureResourceScheduler(size_t simDispatchLanes, size_t deviceSlots, size_t workspaceBudget,
                                  size_t streamCapacity = 0);
  void configurePolicy(const GlobalSchedulerPolicy &policy);
  size_t taskCountInState(GlobalTaskRecord::State state) const;
  SchedulerObservabilitySnapshot observabilitySnapshot() const;

  static BackendCapabilities defaultCapabilitiesForBackend(ExecutionBackendKind backendKind);

private:
  using State = GlobalTaskRecord::State;
  struct TaskEntry {
    RuntimeTask task;
    TaskResourceRequirement needs;
    size_t pendingDependencies = 0;
    std::vector<std::string> dependents;
    State state = State::Submitted;
    std::optional<ResourceReservation> reservation;
    bool waitsForResources = false;
    bool waitsForStreams = false;
    bool waitsForQuota = false;
    ResourceBlockReason blockedBy = ResourceBlockReason::None;
    void clearWaits() {
      waitsForResources = waitsForStreams = waitsForQuota = false;
      blockedBy = ResourceBlockReason::None;
    }
  };
  struct Session {
    ExecutionBackendKind backendKind = ExecutionBackendKind::Host;
    SessionSchedulingOptions scheduling;
    std::map<std::string, TaskEntry> tasks;  // by task id: admission within a session goes in id order
    size_t completed = 0, running = 0, admitted = 0;
    bool failed = false;
    bool quotaReached() const { return scheduling.maxAdmittedTasks > 0 && admitted >= scheduling.maxAdmittedTasks; }
    bool drained() const { return completed == tasks.size() || (failed && running == 0); }
    size_t readyCount() const;
  };
  enum class Attempt { Admitted, NothingReady, QuotaBlocked, ResourceBlocked };

  void admitLocked();                          // admit ready tasks until nothing more fits
  Attempt admitOneLocked(const std::string &sessionId, Session &session);
  void markQuotaWaitLocked(Session &session);
  void giveBackLocked(Session &session, TaskEntry &entry);
  void dropFromRotationLocked(const std::string &sessionId);
  void pointCursorAfterLocked(const std::string &sessionId);
  size_t countStateLocked(State state) const;

  mutable std::mutex mutex_;
  std::condition_variable changed_;
  ResourceScheduler resources_;
  GlobalSchedulerPolicy policy_;
  std::map<std::string, Session> sessions_;
  std::vector<std::string> rotation_;  // session ids in submission order
  size_t cursor_ = 0;                  // where the next admission sweep starts in rotation_
  std::string lastAdmitted_;
  size_t nextOrdinal_ = 0;
  struct Totals {
    int64_t resourceBlocked = 0, streamBlocked = 0, quotaBlocked = 0, reserved = 0, completed = 0, failed = 0,
            sessionsReleased = 0, rotations = 0, skips = 0, turnsTaken = 0;
  } totals_;
};

// The scheduler every ExecutionSession of the process submits to.
GlobalScheduler &globalScheduler();

} // namespace afir
