// Tiny command-line parser for the tools: "--name=value", "--name value", single or double dash, boolean
// flags (the reference tools use llvm::cl, which accepts the same spellings).
#pragma once

#include <map>
#include <set>
#include <string>
#include <vector>

namespace afir {

class CliArgs {
public:
  // `flags` are the boolean options; every other known option takes a value.
  CliArgs(std::set<std::string> valueOptions, std::set<std::string> flags)
      : valueOptions_(std::move(valueOptions)), flags_(std::move(flags)) {}

  bool parse(int argc, char **argv, std::string &error) {
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      if (a.size() < 2 || a[0] != '-') { positional_.push_back(a); continue; }
      a = a.substr(a[1] == '-' ? 2 : 1);
      std::string value;
      bool hasValue = false;
      const size_t eq = a.find('=');
      if (eq != std::string::npos) { value = a.substr(eq + 1); a = a.substr(0, eq); hasValue = true; }
      if (a == "help" || a == "h") { help_ = true; continue; }
      if (flags_.count(a)) {
        values_[a] = hasValue ? value : "true";
        continue;
      }
      if (!valueOptions_.count(a)) { error = "unknown command line argument '" + std::string(argv[i]) + "'"; return false; }
      if (!hasValue) {
        if (i + 1 >= argc) { error = "option '--" + a + "' requires a value"; return false; }
        value = argv[++i];
      }
      values_[a] = value;
    }
    return true;
  }
  bool has(const std::string &name) const { return values_.count(name) != 0; }
  std::string get(const std::string &name, const std::string &dflt = "") const {
    auto it = values_.find(name);
    return it == values_.end() ? dflt : it->second;
  }
  bool flag(const std::string &name) const {
    auto it = values_.find(name);
    return it != values_.end() && it->second != "false" && it->second != "0";
  }
  bool help() const { return help_; }
  const std::vector<std::string> &positional() const { return positional_; }

private:
  std::set<std::string> valueOptions_, flags_;
  std::map<std::string, std::string> values_;
  std::vector<std::string> positional_;
  bool help_ = false;
};

} // namespace afir
