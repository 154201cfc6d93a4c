// A small YAML reader for rack inventories: block mappings and sequences by indentation,
// flow sequences / flow mappings on one line, plain and quoted scalars, comments, and the
// "---" / "..." document markers. Anchors, tags, multi-line scalars and multi-document
// streams are rejected with an error that names the line. The reference project reads the
// same files with yaml-cpp (src/rack_config.cc:96-153); that library is not required here.
#pragma once

#include <string>
#include <utility>
#include <vector>

namespace msharp {

struct YamlNode {
  enum Kind { kNull, kScalar, kSequence, kMapping };
  Kind kind = kNull;
  std::string scalar;
  bool quoted = false;
  int line = 0;
  std::vector<YamlNode> items;                            // kSequence
  std::vector<std::pair<std::string, YamlNode>> entries;  // kMapping, in document order

  bool is_scalar() const { return kind == kScalar; }
  bool is_sequence() const { return kind == kSequence; }
  bool is_mapping() const { return kind == kMapping; }
  const YamlNode* find(const std::string& key) const;  // nullptr when absent or not a mapping
};

// Throws std::runtime_error("yaml: line N: ...") on unsupported or malformed input.
YamlNode parse_yaml(const std::string& text);
YamlNode parse_yaml_file(const std::string& path);  // "cannot read <path>" if unreadable

}  // namespace msharp
