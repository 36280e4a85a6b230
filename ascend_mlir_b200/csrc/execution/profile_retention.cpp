#include "execution/profile_retention.h"

#include <algorithm>
#include <filesystem>
#include <fstream>
#include <vector>

#include "common/json.h"

namespace afir {
namespace fs = std::filesystem;

std::string retainedProfileSessionDirectory(const std::string &root, const std::string &sessionId) {
  return (fs::path(root) / sessionId).string();
}

std::string retainedProfileSessionSummaryPath(const std::string &root, const std::string &sessionId) {
  return (fs::path(root) / sessionId / "session_summary.json").string();
}

Status retainProfileArtifacts(const ProfileTrace &trace, const std::string &root, RetainedProfileArtifacts &out) {
  out.trace = trace;
  const fs::path taskDir = fs::path(retainedProfileSessionDirectory(root, trace.sessionId)) / "tasks";
  std::error_code ec;
  fs::create_directories(taskDir, ec);
  if (ec) return Status::error("cannot create retained profile directory: " + taskDir.string());

  json::Array tasks;
  double total = 0.0;
  std::string backend;
  for (ProfileEvent &ev : out.trace.events) {
    const fs::path kept = taskDir / (ev.taskId + ".json");
    fs::copy_file(ev.artifactPath, kept, fs::copy_options::overwrite_existing, ec);
    if (ec) return Status::error("cannot retain profile artifact " + ev.artifactPath + " -> " + kept.string());
    // the event carries the score; an artifact without one is read back for "score" or "cycle_count"
    double score = ev.score;
    if (score <= 0.0) {
      std::ifstream is(kept);
      std::string text((std::istreambuf_iterator<char>(is)), std::istreambuf_iterator<char>());
      json::Value parsed;
      std::string err;
      if (!json::parse(text, parsed, err))
        return Status::error("cannot parse retained profile artifact for task " + ev.taskId + ": " + err);
      if (!parsed.isObject()) return Status::error("retained profile artifact for task " + ev.taskId + " must be a json object");
      const json::Value *s = parsed.find("score");
      if (!s || !s->isNumber()) s = parsed.find("cycle_count");
      if (!s || !s->isNumber()) return Status::error("retained profile artifact for task " + ev.taskId + " has neither score nor cycle_count");
      score = s->asDouble();
    }
    if (backend.empty()) backend = ev.backend;
    ev.artifactPath = kept.string();
    json::Value t;
    t.set("task_id", ev.taskId);
    t.set("profile_path", ev.artifactPath);
    t.set("score", score);
    t.set("cycle_count", score);
    tasks.push_back(std::move(t));
    total += score;
  }

  json::Value attrs, counters;
  attrs = json::Value(json::Object());
  counters = json::Value(json::Object());
  for (const auto &a : out.trace.attributes) attrs.set(a.first, a.second);
  for (const auto &c : out.trace.counters) counters.set(c.first, c.second);
  json::Value runtime;
  runtime.set("attributes", std::move(attrs));
  runtime.set("counters", std::move(counters));

  const size_t count = tasks.size();
  json::Value root_;
  root_.set("schema_version", 1);
  root_.set("session_id", trace.sessionId);
  root_.set("backend", backend.empty() ? std::string("cuda") : backend);
  root_.set("task_count", static_cast<int64_t>(count));
  root_.set("successful_task_count", static_cast<int64_t>(count));
  root_.set("failed_task_count", 0);
  root_.set("tasks", json::Value(std::move(tasks)));
  root_.set("runtime", std::move(runtime));
  root_.set("total_score", total);
  root_.set("total_cycle_count", total);

  out.summaryPath = retainedProfileSessionSummaryPath(root, trace.sessionId);
  std::ofstream os(out.summaryPath, std::ios::trunc);
  os << json::dump(root_, 2) << "\n";
  os.flush();
  if (!os) return Status::error("cannot write retained session summary: " + out.summaryPath);
  return Status::success();
}

Status pruneRetainedProfileDirectories(const std::string &root, size_t keepCount) {
  std::error_code ec;
  if (!fs::exists(root, ec)) return Status::success();
  struct Entry {
    std::string path;
    fs::file_time_type mtime;
  };
  std::vector<Entry> dirs;
  fs::directory_iterator it(root, ec), end;
  if (ec) return Status::error("cannot iterate retained profile root: " + root);
  for (; it != end; it.increment(ec)) {
    if (ec) return Status::error("cannot iterate retained profile root: " + root);
    std::error_code e2;
    if (!it->is_directory(e2) || e2) continue;
    auto mtime = fs::last_write_time(it->path(), e2);
    if (e2) mtime = fs::file_time_type::min();
    dirs.push_back({it->path().string(), mtime});
  }
  if (dirs.size() <= keepCount) return Status::success();
  std::sort(dirs.begin(), dirs.end(), [](const Entry &a, const Entry &b) { return a.mtime != b.mtime ? a.mtime > b.mtime : a.path < b.path; });
  for (size_t i = keepCount; i < dirs.size(); ++i) {
    std::error_code e2;
    fs::remove_all(dirs[i].path, e2);  // best effort: a directory that cannot be removed is tried again next time
  }
  return Status::success();
}

Status prepareRetainedRootForNewSession(const std::string &root, size_t sessionLimit) {
  std::error_code ec;
  fs::create_directories(root, ec);
  if (ec) return Status::error("cannot create retained profile directory: " + root);
  return pruneRetainedProfileDirectories(root, pruneKeepCountForNewSession(sessionLimit));
}

} // namespace afir
