#include "execution/task_graph.h"

#include <queue>
#include <unordered_map>

namespace afir {

Status TaskGraph::addTask(const RuntimeTask &task) {
  if (task.taskId.empty()) return Status::error("empty task id");
  for (const auto &t : tasks_)
    if (t.taskId == task.taskId) return Status::error("duplicate task id");
  tasks_.push_back(task);
  return Status::success();
}

Status TaskGraph::orderedTasks(std::vector<RuntimeTask> &order) const {
  order.clear();
  std::unordered_map<std::string, size_t> index;
  for (size_t i = 0; i < tasks_.size(); ++i) index.emplace(tasks_[i].taskId, i);
  std::vector<size_t> indegree(tasks_.size(), 0);
  std::vector<std::vector<size_t>> out(tasks_.size());
  for (size_t i = 0; i < tasks_.size(); ++i)
    for (const auto &dep : tasks_[i].dependencies) {
      auto it = index.find(dep);
      if (it == index.end()) return Status::error("unknown task dependency");
      out[it->second].push_back(i);
      ++indegree[i];
    }
  std::queue<size_t> ready;
  for (size_t i = 0; i < tasks_.size(); ++i)
    if (indegree[i] == 0) ready.push(i);
  while (!ready.empty()) {
    const size_t i = ready.front();
    ready.pop();
    order.push_back(tasks_[i]);
    for (size_t n : out[i])
      if (--indegree[n] == 0) ready.push(n);
  }
  if (order.size() != tasks_.size()) return Status::error("task graph contains a cycle");
  return Status::success();
}

Status TaskGraph::topologicalOrder(std::vector<std::string> &ids) const {
  std::vector<RuntimeTask> order;
  if (Status s = orderedTasks(order); !s) return s;
  ids.clear();
  for (const auto &t : order) ids.push_back(t.taskId);
  return Status::success();
}

} // namespace afir
