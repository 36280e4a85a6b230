// Capacity accounting for task admission on one node: how many launch lanes, GPUs ("device slots"), CUDA
// streams ("stream units") and bytes of device scratch the admitted tasks hold together.  A task is admitted
// only when every resource it asks for fits; the grant is returned as a reservation that must be handed
// back.  Interface and blocking rules follow the reference's include/Runtime/Execution/ResourceScheduler.h
// and lib/Runtime/Execution/ResourceScheduler.cpp:24-153; the backend kinds are re-hosted: "Host" is a
// backend whose launches go through serialised lanes (the reference's simulator), "Cuda" one that occupies
// GPUs (the reference's NPU).
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <optional>
#include <string>

namespace afir {

enum class ExecutionBackendKind { Host, Cuda };

enum class ResourceBlockReason {
  None,
  Workspace,
  SerializedLaunch,
  DeviceCapacity,
  StreamCapacity,
  ExclusiveStreamConflict,
};
const char *resourceBlockReasonName(ResourceBlockReason reason);

struct TaskResourceRequirement {
  ExecutionBackendKind backendKind = ExecutionBackendKind::Host;
  size_t workspaceBytes = 0;
  bool requiresSerializedLaunch = false;  // Host backends only: one lane per running task
  bool exclusiveDeviceAccess = false;     // Cuda backends only: the task takes every GPU
  bool requiresStream = false;
  size_t streamUnits = 0;                 // 0 with requiresStream/exclusiveStreamAccess counts as 1
  bool exclusiveStreamAccess = false;     // no other stream holder may run beside this task
};

struct ResourceReservation {
  std::string sessionId;
  std::string taskId;
  ExecutionBackendKind backendKind = ExecutionBackendKind::Host;
  size_t workspaceBytes = 0;
  bool holdsSerializedLaunchLane = false;
  bool holdsDeviceSlot = false;
  bool holdsStreamSlot = false;
  size_t reservedStreamUnits = 0;

private:
  friend class ResourceScheduler;
  uint64_t ticket_ = 0;  // issued by the scheduler; a reservation rebuilt from its public fields has none
};

class ResourceScheduler {
public:
  void configureSimDispatchLanes(size_t count) { limit_.lanes = count; }
  void configureDeviceSlots(size_t count) { limit_.devices = count; }
  void configureWorkspaceBudget(size_t bytes) { limit_.workspace = bytes; }
  void configureStreamCapacity(size_t count) { limit_.streams = count; }

  ResourceBlockReason lastBlockReason() const { return lastBlock_; }
  size_t configuredStreamCapacity() const { return limit_.streams; }
  size_t reservedStreamUnits() const { return held_.streams; }
  size_t availableStreamCapacity() const { return limit_.streams > held_.streams ? limit_.streams - held_.streams : 0; }
  size_t reservedDeviceSlots() const { return held_.devices; }
  size_t reservedWorkspaceBytes() const { return held_.workspace; }
  size_t activeReservationCount() const { return grants_.size(); }

  // Admits the task or says why not (lastBlockReason()).  Nothing is held after a refusal.
  std::optional<ResourceReservation> tryReserve(const std::string &sessionId, const std::string &taskId,
                                                const TaskResourceRequirement &requirement);
  // Hands a grant back.  Unknown, stale or hand-built reservations are ignored.
  void release(const ResourceReservation &reservation);

private:
  struct Amounts {
    size_t lanes = 0, devices = 0, workspace = 0, streams = 0;
  };
  struct Grant {
    ResourceReservation issued;
    Amounts amounts;
    bool exclusiveStreams = false;
  };
  Amounts limit_{1, 1, 0, 0};
  Amounts held_;
  bool exclusiveStreamHolder_ = false;
  ResourceBlockReason lastBlock_ = ResourceBlockReason::None;
  uint64_t nextTicket_ = 1;
  std::map<uint64_t, Grant> grants_;
};

} // namespace afir
