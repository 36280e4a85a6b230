// Keeps the profile artifacts of a finished session where they outlive the session directory:
// <root>/<session id>/tasks/<task id>.json (copies of each task's trace.json) and
// <root>/<session id>/session_summary.json (tasks with their scores, the session's runtime attributes and
// counters, totals).  Old sessions are pruned by directory age so that at most `sessionLimit` remain.
// Layout, key names and pruning rule follow the reference's lib/Runtime/Profile/ProfileUtils.cpp:123-448;
// scores here are kernel microseconds (floating point), not simulator cycle counts.
#pragma once

#include <string>

#include "execution/execution_session.h"

namespace afir {

struct RetainedProfileArtifacts {
  ProfileTrace trace;        // the session's trace with every event pointing at its retained copy
  std::string summaryPath;   // <root>/<session id>/session_summary.json
};

std::string retainedProfileSessionDirectory(const std::string &root, const std::string &sessionId);
std::string retainedProfileSessionSummaryPath(const std::string &root, const std::string &sessionId);

Status retainProfileArtifacts(const ProfileTrace &trace, const std::string &root, RetainedProfileArtifacts &out);

// Removes all but the `keepCount` most recently modified directories directly under `root` (ties: by path).
// A missing root is fine.  Plain files are left alone.
Status pruneRetainedProfileDirectories(const std::string &root, size_t keepCount);

// Before a new session writes under `root`: create it and prune to sessionLimit - 1 directories.
inline size_t pruneKeepCountForNewSession(size_t sessionLimit) { return sessionLimit > 0 ? sessionLimit - 1 : 0; }
Status prepareRetainedRootForNewSession(const std::string &root, size_t sessionLimit);

} // namespace afir
