#include "msharp/rack.h"

#include <cerrno>
#include <climits>
#include <cstdlib>
#include <set>
#include <sstream>
#include <stdexcept>

#include "msharp/json.h"
#include "msharp/yaml_lite.h"

namespace msharp {
namespace {

bool scalar_to_int(const YamlNode& node, int* out) {
  if (!node.is_scalar() || node.scalar.empty()) {
    return false;
  }
  errno = 0;
  char* end = nullptr;
  const long v = std::strtol(node.scalar.c_str(), &end, 0);
  if (*end != '\0' || errno == ERANGE || v > INT_MAX || v < INT_MIN) {
    return false;
  }
  *out = static_cast<int>(v);
  return true;
}

// The body of a tray: a mapping as is, or a sequence of mappings merged left to right.
YamlNode merged_body(const YamlNode& body, const std::string& label) {
  if (body.is_mapping()) {
    return body;
  }
  if (!body.is_sequence()) {
    throw std::runtime_error("rack entry " + label + " must be a map or sequence of maps");
  }
  YamlNode merged;
  merged.kind = YamlNode::kMapping;
  for (const YamlNode& part : body.items) {
    if (!part.is_mapping()) {
      throw std::runtime_error("rack entry " + label + " sequence items must be maps");
    }
    for (const auto& field : part.entries) {
      bool replaced = false;
      for (auto& existing : merged.entries) {
        if (existing.first == field.first) {
          existing.second = field.second;
          replaced = true;
        }
      }
      if (!replaced) {
        merged.entries.push_back(field);
      }
    }
  }
  return merged;
}

RackEntry entry_from_item(const YamlNode& item) {
  if (!item.is_mapping() || item.entries.size() != 1) {
    throw std::runtime_error("each rack item must be a single-key map");
  }
  RackEntry entry;
  entry.host_label = item.entries[0].first;
  if (entry.host_label.empty()) {
    throw std::runtime_error("rack entry host label cannot be empty");
  }
  const std::string& label = entry.host_label;
  const YamlNode body = merged_body(item.entries[0].second, label);

  const YamlNode* hostname = body.find("hostname");
  if (hostname == nullptr || !hostname->is_scalar()) {
    throw std::runtime_error("rack entry " + label + " requires scalar field 'hostname'");
  }
  entry.control_hostname = hostname->scalar;

  if (const YamlNode* port = body.find("port"); port != nullptr && port->kind != YamlNode::kNull) {
    if (!port->is_scalar()) {
      throw std::runtime_error("rack entry " + label + " field 'port' must be scalar");
    }
    if (!scalar_to_int(*port, &entry.ssh_port)) {
      throw std::runtime_error("rack entry " + label + " has invalid SSH port");
    }
  }
  if (entry.ssh_port <= 0 || entry.ssh_port > 65535) {
    throw std::runtime_error("rack entry " + label + " has invalid SSH port");
  }

  const YamlNode* device = body.find("device");
  if (device == nullptr || !device->is_sequence()) {
    throw std::runtime_error("rack entry " + label + " requires 'device' as a YAML sequence");
  }
  std::set<int> seen;
  for (const YamlNode& d : device->items) {
    int ordinal = 0;
    if (!scalar_to_int(d, &ordinal)) {
      throw std::runtime_error("rack entry " + label + " device entries must be scalar integers");
    }
    if (ordinal < 0) {
      throw std::runtime_error("rack entry " + label + " lists a negative CUDA device ordinal");
    }
    if (!seen.insert(ordinal).second) {
      throw std::runtime_error("rack entry " + label + " lists duplicate CUDA device ordinals");
    }
    entry.devices.push_back(ordinal);
  }
  if (entry.devices.empty() || static_cast<int>(entry.devices.size()) > kMaxDevicesPerTray) {
    throw std::runtime_error("rack entry " + label + " must list 1 to " + std::to_string(kMaxDevicesPerTray) +
                             " CUDA device ordinals");
  }
  return entry;
}

void validate_entries(const std::vector<RackEntry>& entries) {
  if (entries.empty() || static_cast<int>(entries.size()) > kMaxTrays) {
    throw std::runtime_error("rack config must contain 1 to " + std::to_string(kMaxTrays) + " rack entries");
  }
  std::size_t total = 0;
  for (const auto& e : entries) {
    total += e.devices.size();
  }
  if (total > static_cast<std::size_t>(kMaxRanks)) {
    throw std::runtime_error("rack config describes more than " + std::to_string(kMaxRanks) + " CUDA devices");
  }
}

void entries_from_root(const YamlNode& root, std::vector<RackEntry>* sink) {
  const YamlNode* rack = root.find("rack");
  if (rack == nullptr || !rack->is_sequence()) {
    throw std::runtime_error("rack config must contain a top-level sequence named 'rack'");
  }
  std::set<std::string> labels;
  for (const YamlNode& item : rack->items) {
    RackEntry entry = entry_from_item(item);
    if (!labels.insert(normalize_host_label(entry.host_label)).second) {
      throw std::runtime_error("duplicate rack host label: " + entry.host_label);
    }
    sink->push_back(std::move(entry));
  }
  validate_entries(*sink);
}

}  // namespace

std::string normalize_host_label(const std::string& host) { return host.substr(0, host.find('.')); }

const RankTarget& RankPlan::target(int rank) const {
  if (rank < 0 || rank >= size()) {
    throw std::runtime_error("rank index is outside the selected rank plan");
  }
  return targets_[static_cast<std::size_t>(rank)];
}

int RankPlan::slot_count_for_host(const std::string& host_label) const {
  const std::string wanted = normalize_host_label(host_label);
  int count = 0;
  for (const auto& t : targets_) {
    count += normalize_host_label(t.host_label) == wanted;
  }
  return count;
}

std::map<std::string, int> RankPlan::slot_counts_by_host() const {
  std::map<std::string, int> counts;
  for (const auto& t : targets_) {
    ++counts[normalize_host_label(t.host_label)];
  }
  return counts;
}

std::map<std::string, std::vector<int>> RankPlan::devices_by_host() const {
  std::map<std::string, std::vector<int>> devices;
  for (const auto& t : targets_) {
    devices[normalize_host_label(t.host_label)].push_back(t.gpu_ordinal);
  }
  return devices;
}

int RankPlan::local_rank(int rank) const {
  const std::string host = normalize_host_label(target(rank).host_label);
  int local = 0;
  for (int r = 0; r < rank; ++r) {
    local += normalize_host_label(targets_[static_cast<std::size_t>(r)].host_label) == host;
  }
  return local;
}

RackConfig RackConfig::load(const std::string& path) {
  RackConfig cfg;
  entries_from_root(parse_yaml_file(path), &cfg.entries_);
  return cfg;
}

RackConfig RackConfig::parse(const std::string& yaml_text) {
  RackConfig cfg;
  entries_from_root(parse_yaml(yaml_text), &cfg.entries_);
  return cfg;
}

RackConfig RackConfig::single_host(const std::string& label, int device_count) {
  RackConfig cfg;
  RackEntry e;
  e.host_label = label;
  e.control_hostname = "127.0.0.1";
  for (int d = 0; d < device_count; ++d) {
    e.devices.push_back(d);
  }
  if (e.devices.empty() || device_count > kMaxDevicesPerTray) {
    throw std::runtime_error("rack entry " + label + " must list 1 to " + std::to_string(kMaxDevicesPerTray) +
                             " CUDA device ordinals");
  }
  cfg.entries_.push_back(e);
  return cfg;
}

const RackEntry* RackConfig::find_by_host_label(const std::string& label) const {
  const int idx = index_of_host_label(label);
  return idx < 0 ? nullptr : &entries_[static_cast<std::size_t>(idx)];
}

int RackConfig::index_of_host_label(const std::string& label) const {
  const std::string wanted = normalize_host_label(label);
  for (std::size_t i = 0; i < entries_.size(); ++i) {
    if (normalize_host_label(entries_[i].host_label) == wanted) {
      return static_cast<int>(i);
    }
  }
  return -1;
}

std::size_t RackConfig::available_rank_count() const {
  std::size_t total = 0;
  for (const auto& e : entries_) {
    total += e.devices.size();
  }
  return total;
}

std::string RackConfig::to_yaml() const {
  std::ostringstream os;
  os << "rack:\n";
  for (const auto& e : entries_) {
    os << "  - " << e.host_label << ":\n";
    os << "      - hostname: " << e.control_hostname << "\n";
    os << "      - port: " << e.ssh_port << "\n";
    os << "      - device: [";
    for (std::size_t i = 0; i < e.devices.size(); ++i) {
      os << (i ? ", " : "") << e.devices[i];
    }
    os << "]\n";
  }
  return os.str();
}

RankPlan build_rank_plan(const RackConfig& rack, int rank_count, const std::string& selection) {
  if (rank_count <= 0) {
    throw std::runtime_error("rank_count must be positive");
  }
  const std::size_t available = rack.available_rank_count();
  if (static_cast<std::size_t>(rank_count) > available) {
    throw std::runtime_error("rank_count " + std::to_string(rank_count) + " exceeds rack.yaml device count " +
                             std::to_string(available));
  }
  const bool prefix = selection == "prefix";
  if (!prefix && selection != "balanced") {
    throw std::runtime_error("rank selection must be balanced or prefix");
  }

  // Enumerate (tray, slot) pairs in the order of the policy and keep the first rank_count.
  const auto& trays = rack.entries();
  std::vector<RankTarget> targets;
  auto take = [&](std::size_t tray, std::size_t slot) {
    const RackEntry& e = trays[tray];
    RankTarget t;
    t.rank_index_in_plan = static_cast<int>(targets.size());
    t.rack_index = static_cast<int>(tray);
    t.host_label = e.host_label;
    t.control_hostname = e.control_hostname;
    t.ssh_port = e.ssh_port;
    t.gpu_ordinal = e.devices[slot];
    targets.push_back(std::move(t));
  };
  const std::size_t outer = prefix ? trays.size() : static_cast<std::size_t>(kMaxDevicesPerTray);
  const std::size_t inner = prefix ? static_cast<std::size_t>(kMaxDevicesPerTray) : trays.size();
  for (std::size_t a = 0; a < outer && static_cast<int>(targets.size()) < rank_count; ++a) {
    for (std::size_t b = 0; b < inner && static_cast<int>(targets.size()) < rank_count; ++b) {
      const std::size_t tray = prefix ? a : b;
      const std::size_t slot = prefix ? b : a;
      if (slot < trays[tray].devices.size()) {
        take(tray, slot);
      }
    }
  }
  if (static_cast<int>(targets.size()) != rank_count) {
    throw std::runtime_error("failed to build a complete rank plan");
  }
  return RankPlan(std::move(targets));
}

namespace {

// Labels of selected trays in first-use order, with their rank counts.
std::vector<std::pair<std::string, int>> ordered_counts(const RankPlan& plan) {
  std::vector<std::pair<std::string, int>> counts;
  for (const auto& t : plan.targets()) {
    bool found = false;
    for (auto& c : counts) {
      if (c.first == t.host_label) {
        ++c.second;
        found = true;
      }
    }
    if (!found) {
      counts.emplace_back(t.host_label, 1);
    }
  }
  return counts;
}

bool selected(const RankPlan& plan, const std::string& label) {
  for (const auto& t : plan.targets()) {
    if (t.host_label == label) {
      return true;
    }
  }
  return false;
}

}  // namespace

std::string host_list_text(const RankPlan& plan) {
  std::ostringstream os;
  bool first = true;
  for (const auto& c : ordered_counts(plan)) {
    os << (first ? "" : ",") << c.first << ":" << c.second;
    first = false;
  }
  return os.str();
}

std::string rankfile_text(const RankPlan& plan) {
  std::ostringstream os;
  for (int r = 0; r < plan.size(); ++r) {
    os << "rank " << r << "=" << plan.target(r).host_label << " slot=" << plan.local_rank(r) << "\n";
  }
  return os.str();
}

std::string selected_entries_text(const RackConfig& rack, const RankPlan& plan) {
  std::ostringstream os;
  for (const auto& e : rack.entries()) {
    if (selected(plan, e.host_label)) {
      os << e.host_label << "\t" << e.control_hostname << "\t" << e.ssh_port << "\n";
    }
  }
  return os.str();
}

std::string ssh_config_text(const RackConfig& rack, const RankPlan& plan, const SshOptions& opt) {
  std::ostringstream os;
  for (const auto& e : rack.entries()) {
    if (!selected(plan, e.host_label)) {
      continue;
    }
    os << "Host " << e.host_label << "\n"
       << "  HostName " << e.control_hostname << "\n"
       << "  User " << opt.user << "\n"
       << "  Port " << e.ssh_port << "\n"
       << "  IdentityFile " << opt.identity << "\n"
       << "  IdentitiesOnly yes\n"
       << "  PasswordAuthentication no\n"
       << "  UserKnownHostsFile " << opt.known_hosts << "\n"
       << "  StrictHostKeyChecking accept-new\n"
       << "  BatchMode yes\n\n";
  }
  return os.str();
}

std::string rack_to_json(const RackConfig& rack) {
  JsonWriter w;
  w.begin_object();
  w.key("available_rank_count").value(static_cast<uint64_t>(rack.available_rank_count()));
  w.key("entries").begin_array();
  for (const auto& e : rack.entries()) {
    w.begin_object();
    w.key("host_label").value(e.host_label);
    w.key("hostname").value(e.control_hostname);
    w.key("port").value(e.ssh_port);
    w.key("devices").begin_array();
    for (int d : e.devices) {
      w.value(d);
    }
    w.end_array();
    w.end_object();
  }
  w.end_array();
  w.end_object();
  return w.str();
}

std::string plan_to_json(const RankPlan& plan) {
  JsonWriter w;
  w.begin_array();
  for (int r = 0; r < plan.size(); ++r) {
    const RankTarget& t = plan.target(r);
    w.begin_object();
    w.key("rank").value(t.rank_index_in_plan);
    w.key("rack_index").value(t.rack_index);
    w.key("host_label").value(t.host_label);
    w.key("hostname").value(t.control_hostname);
    w.key("port").value(t.ssh_port);
    w.key("gpu").value(t.gpu_ordinal);
    w.key("local_rank").value(plan.local_rank(r));
    w.end_object();
  }
  w.end_array();
  return w.str();
}

}  // namespace msharp
