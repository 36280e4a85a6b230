#include "execution/resource_scheduler.h"

#include <algorithm>

namespace afir {

const char *resourceBlockReasonName(ResourceBlockReason reason) {
  switch (reason) {
  case ResourceBlockReason::None: return "none";
  case ResourceBlockReason::Workspace: return "workspace";
  case ResourceBlockReason::SerializedLaunch: return "serialized_launch";
  case ResourceBlockReason::DeviceCapacity: return "device_capacity";
  case ResourceBlockReason::StreamCapacity: return "stream_capacity";
  case ResourceBlockReason::ExclusiveStreamConflict: return "exclusive_stream_conflict";
  }
  return "none";
}

std::optional<ResourceReservation> ResourceScheduler::tryReserve(const std::string &sessionId, const std::string &taskId,
                                                                 const TaskResourceRequirement &req) {
  // What the task would hold if admitted.
  Amounts want;
  want.workspace = req.workspaceBytes;
  if (req.backendKind == ExecutionBackendKind::Host && req.requiresSerializedLaunch) want.lanes = 1;
  if (req.backendKind == ExecutionBackendKind::Cuda) want.devices = req.exclusiveDeviceAccess ? limit_.devices : 1;
  const bool wantsStream = req.requiresStream || req.streamUnits > 0 || req.exclusiveStreamAccess;
  if (wantsStream) want.streams = std::max<size_t>(req.streamUnits, 1);

  // First resource that does not fit, in a fixed order (scratch, lane, GPU, stream).  A budget lowered
  // below what is already out blocks everything until enough comes back.
  auto refusal = [&]() {
    if (limit_.workspace < held_.workspace || want.workspace > limit_.workspace - held_.workspace)
      return ResourceBlockReason::Workspace;
    if (want.lanes && limit_.lanes <= held_.lanes) return ResourceBlockReason::SerializedLaunch;
    if (req.backendKind == ExecutionBackendKind::Cuda &&
        (want.devices == 0 || limit_.devices < held_.devices + want.devices))
      return ResourceBlockReason::DeviceCapacity;
    if (want.streams) {
      const bool othersHoldStreams = held_.streams > 0 || exclusiveStreamHolder_;
      if (req.exclusiveStreamAccess ? othersHoldStreams : exclusiveStreamHolder_)
        return ResourceBlockReason::ExclusiveStreamConflict;
      if (limit_.streams < held_.streams + want.streams) return ResourceBlockReason::StreamCapacity;
    }
    return ResourceBlockReason::None;
  };
  lastBlock_ = refusal();
  if (lastBlock_ != ResourceBlockReason::None) return std::nullopt;

  Grant grant;
  grant.amounts = want;
  grant.exclusiveStreams = want.streams > 0 && req.exclusiveStreamAccess;
  ResourceReservation &r = grant.issued;
  r.sessionId = sessionId;
  r.taskId = taskId;
  r.backendKind = req.backendKind;
  r.workspaceBytes = want.workspace;
  r.holdsSerializedLaunchLane = want.lanes > 0;
  r.holdsDeviceSlot = want.devices > 0;
  r.holdsStreamSlot = want.streams > 0;
  r.reservedStreamUnits = want.streams;
  r.ticket_ = nextTicket_++;

  held_.workspace += want.workspace;
  held_.lanes += want.lanes;
  held_.devices += want.devices;
  held_.streams += want.streams;
  exclusiveStreamHolder_ = exclusiveStreamHolder_ || grant.exclusiveStreams;
  const ResourceReservation issued = r;
  grants_.emplace(issued.ticket_, std::move(grant));
  return issued;
}

void ResourceScheduler::release(const ResourceReservation &r) {
  auto it = grants_.find(r.ticket_);
  if (it == grants_.end()) return;
  const ResourceReservation &live = it->second.issued;
  const bool sameGrant = live.sessionId == r.sessionId && live.taskId == r.taskId && live.backendKind == r.backendKind &&
                         live.workspaceBytes == r.workspaceBytes &&
                         live.holdsSerializedLaunchLane == r.holdsSerializedLaunchLane &&
                         live.holdsDeviceSlot == r.holdsDeviceSlot && live.holdsStreamSlot == r.holdsStreamSlot &&
                         live.reservedStreamUnits == r.reservedStreamUnits;
  if (!sameGrant) return;
  const Amounts back = it->second.amounts;
  if (it->second.exclusiveStreams) exclusiveStreamHolder_ = false;
  grants_.erase(it);
  held_.workspace -= back.workspace;
  held_.lanes -= back.lanes;
  held_.devices -= back.devices;
  held_.streams -= back.streams;
  lastBlock_ = ResourceBlockReason::None;
}

} // namespace afir
