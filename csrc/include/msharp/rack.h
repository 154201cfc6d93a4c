// Rack inventory (YAML) and deterministic rank plan.
//
// Behaviour follows the reference project (paths within it):
//   src/rack_config.cc:24-50   a tray body is a mapping, or a sequence of one-key maps that is merged
//   src/rack_config.cc:96-153  field rules: unique labels after short-name normalisation, scalar
//                              "hostname", optional "port" (default 4399, 1..65535), "device" is a
//                              YAML sequence of unique non-negative integers
//   src/rack_config.cc:172-224 "prefix" (tray order, listed device order) and "balanced"
//                              (device slot 0 of every tray, then slot 1, ...) plans
//   scripts/run_mnnvl_sharp.sh:184-216  host list, ssh config, entries table and rankfile texts
// Difference: a tray may list up to 8 devices (the reference stops at 4) so that one
// 8-GPU HGX baseboard can be described as a single tray; 18 trays / 72 devices stay the caps.
#pragma once

#include <cstddef>
#include <map>
#include <string>
#include <vector>

namespace msharp {

constexpr int kMaxDevicesPerTray = 8;
constexpr int kMaxTrays = 18;
constexpr int kMaxRanks = 72;
constexpr int kDefaultSshPort = 4399;

struct RackEntry {
  std::string host_label;
  std::string control_hostname;
  int ssh_port = kDefaultSshPort;
  std::vector<int> devices;
};

struct RankTarget {
  int rank_index_in_plan = -1;
  int rack_index = -1;
  std::string host_label;
  std::string control_hostname;
  int ssh_port = kDefaultSshPort;
  int gpu_ordinal = -1;
};

std::string normalize_host_label(const std::string& host);  // strip from the first '.'

class RankPlan {
 public:
  RankPlan() = default;
  explicit RankPlan(std::vector<RankTarget> targets) : targets_(std::move(targets)) {}

  const std::vector<RankTarget>& targets() const { return targets_; }
  int size() const { return static_cast<int>(targets_.size()); }
  const RankTarget& target(int rank) const;  // throws when out of range
  int slot_count_for_host(const std::string& host_label) const;
  std::map<std::string, int> slot_counts_by_host() const;
  std::map<std::string, std::vector<int>> devices_by_host() const;
  // index of `rank` among the ranks of its own host (the "local rank" / rankfile slot)
  int local_rank(int rank) const;

 private:
  std::vector<RankTarget> targets_;
};

class RackConfig {
 public:
  static RackConfig load(const std::string& path);
  static RackConfig parse(const std::string& yaml_text);
  // One tray named `label` with devices 0..device_count-1 (used when no YAML is given).
  static RackConfig single_host(const std::string& label, int device_count);

  const std::vector<RackEntry>& entries() const { return entries_; }
  const RackEntry* find_by_host_label(const std::string& label) const;
  int index_of_host_label(const std::string& label) const;  // -1 when absent
  std::size_t available_rank_count() const;
  std::string to_yaml() const;

 private:
  std::vector<RackEntry> entries_;
};

RankPlan build_rank_plan(const RackConfig& rack, int rank_count, const std::string& selection);

// Launch artefacts (pure text producers).
struct SshOptions {
  std::string user = "ubuntu";
  std::string identity = "/home/ubuntu/.ssh/id_rsa";
  std::string known_hosts = "/home/ubuntu/.ssh/known_hosts";
};
std::string host_list_text(const RankPlan& plan);                        // "label:count,label:count"
std::string rankfile_text(const RankPlan& plan);                         // "rank R=label slot=S" lines
std::string selected_entries_text(const RackConfig& rack, const RankPlan& plan);  // label \t host \t port
std::string ssh_config_text(const RackConfig& rack, const RankPlan& plan, const SshOptions& opt);

std::string rack_to_json(const RackConfig& rack);
std::string plan_to_json(const RankPlan& plan);

}  // namespace msharp
