#include "msharp/yaml_lite.h"

#include <fstream>
#include <sstream>
#include <stdexcept>

namespace msharp {
namespace {

struct Line {
  int indent = 0;
  std::string text;  // without indentation, comment and trailing blanks
  int number = 0;
};

[[noreturn]] void fail(int line, const std::string& what) {
  throw std::runtime_error("yaml: line " + std::to_string(line) + ": " + what);
}

// Remove a trailing comment (a '#' at the start or preceded by a blank, outside quotes).
std::string strip_comment(const std::string& s) {
  char quote = 0;
  for (std::size_t i = 0; i < s.size(); ++i) {
    const char c = s[i];
    if (quote) {
      if (c == quote) {
        quote = 0;
      } else if (c == '\\' && quote == '"') {
        ++i;
      }
    } else if (c == '"' || c == '\'') {
      quote = c;
    } else if (c == '#' && (i == 0 || s[i - 1] == ' ' || s[i - 1] == '\t')) {
      return s.substr(0, i);
    }
  }
  return s;
}

std::string rtrim(std::string s) {
  while (!s.empty() && (s.back() == ' ' || s.back() == '\t' || s.back() == '\r')) {
    s.pop_back();
  }
  return s;
}

std::string trim(const std::string& s) {
  std::size_t b = 0;
  while (b < s.size() && (s[b] == ' ' || s[b] == '\t')) {
    ++b;
  }
  return rtrim(s.substr(b));
}

std::vector<Line> split_lines(const std::string& text) {
  std::vector<Line> lines;
  std::istringstream in(text);
  std::string raw;
  int number = 0;
  bool seen_document = false;
  while (std::getline(in, raw)) {
    ++number;
    std::string body = rtrim(strip_comment(raw));
    if (body.empty()) {
      continue;
    }
    std::size_t indent = 0;
    while (indent < body.size() && body[indent] == ' ') {
      ++indent;
    }
    if (indent < body.size() && body[indent] == '\t') {
      fail(number, "tab characters cannot be used for indentation");
    }
    std::string content = body.substr(indent);
    if (content.empty()) {
      continue;
    }
    if (indent == 0 && (content == "---" || content == "...")) {
      if (content == "---" && seen_document && !lines.empty()) {
        fail(number, "multiple documents are not supported");
      }
      seen_document = true;
      continue;
    }
    if (content[0] == '%') {
      continue;  // directive
    }
    lines.push_back(Line{static_cast<int>(indent), content, number});
  }
  return lines;
}

// Position of the ':' that separates key and value on this line, or npos.
std::size_t key_separator(const std::string& s) {
  char quote = 0;
  int depth = 0;
  for (std::size_t i = 0; i < s.size(); ++i) {
    const char c = s[i];
    if (quote) {
      if (c == quote) {
        quote = 0;
      } else if (c == '\\' && quote == '"') {
        ++i;
      }
      continue;
    }
    if (c == '"' || c == '\'') {
      quote = c;
    } else if (c == '[' || c == '{') {
      ++depth;
    } else if (c == ']' || c == '}') {
      --depth;
    } else if (c == ':' && depth == 0 && (i + 1 == s.size() || s[i + 1] == ' ' || s[i + 1] == '\t')) {
      return i;
    }
  }
  return std::string::npos;
}

YamlNode make_scalar(const std::string& token, int line) {
  YamlNode n;
  n.line = line;
  const std::string t = trim(token);
  if (t.empty() || t == "~" || t == "null") {
    n.kind = YamlNode::kNull;
    return n;
  }
  if (t[0] == '&' || t[0] == '*' || t[0] == '!' || t[0] == '|' || t[0] == '>') {
    fail(line, "anchors, aliases, tags and block scalars are not supported");
  }
  n.kind = YamlNode::kScalar;
  if (t.size() >= 2 && (t[0] == '"' || t[0] == '\'') && t.back() == t[0]) {
    n.quoted = true;
    const char q = t[0];
    for (std::size_t i = 1; i + 1 < t.size(); ++i) {
      if (q == '"' && t[i] == '\\' && i + 2 < t.size()) {
        const char e = t[++i];
        n.scalar += e == 'n' ? '\n' : e == 't' ? '\t' : e;
      } else if (q == '\'' && t[i] == '\'' && i + 2 < t.size() && t[i + 1] == '\'') {
        n.scalar += '\'';
        ++i;
      } else {
        n.scalar += t[i];
      }
    }
  } else {
    if (t[0] == '"' || t[0] == '\'') {
      fail(line, "unterminated quoted scalar");
    }
    n.scalar = t;
  }
  return n;
}

// Flow collections on a single line: [a, b, [c]] and {k: v, ...}.
class FlowParser {
 public:
  FlowParser(const std::string& s, int line) : s_(s), line_(line) {}

  YamlNode parse_all() {
    YamlNode n = parse_value();
    skip_blanks();
    if (pos_ != s_.size()) {
      fail(line_, "unexpected text after flow collection");
    }
    return n;
  }

 private:
  void skip_blanks() {
    while (pos_ < s_.size() && (s_[pos_] == ' ' || s_[pos_] == '\t')) {
      ++pos_;
    }
  }

  YamlNode parse_value() {
    skip_blanks();
    if (pos_ >= s_.size()) {
      fail(line_, "unterminated flow collection");
    }
    if (s_[pos_] == '[') {
      return parse_sequence();
    }
    if (s_[pos_] == '{') {
      return parse_mapping();
    }
    return make_scalar(take_token(",]}"), line_);
  }

  std::string take_token(const char* stops) {
    std::string tok;
    char quote = 0;
    while (pos_ < s_.size()) {
      const char c = s_[pos_];
      if (quote) {
        tok += c;
        if (c == quote) {
          quote = 0;
        }
      } else if (c == '"' || c == '\'') {
        quote = c;
        tok += c;
      } else if (std::string(stops).find(c) != std::string::npos) {
        break;
      } else {
        tok += c;
      }
      ++pos_;
    }
    return tok;
  }

  YamlNode parse_sequence() {
    YamlNode n;
    n.kind = YamlNode::kSequence;
    n.line = line_;
    ++pos_;  // [
    skip_blanks();
    if (pos_ < s_.size() && s_[pos_] == ']') {
      ++pos_;
      return n;
    }
    for (;;) {
      n.items.push_back(parse_value());
      skip_blanks();
      if (pos_ >= s_.size()) {
        fail(line_, "flow sequence must be closed on the same line");
      }
      if (s_[pos_] == ',') {
        ++pos_;
        skip_blanks();
        if (pos_ < s_.size() && s_[pos_] == ']') {  // trailing comma
          ++pos_;
          return n;
        }
        continue;
      }
      if (s_[pos_] == ']') {
        ++pos_;
        return n;
      }
      fail(line_, "expected ',' or ']' in flow sequence");
    }
  }

  YamlNode parse_mapping() {
    YamlNode n;
    n.kind = YamlNode::kMapping;
    n.line = line_;
    ++pos_;  // {
    skip_blanks();
    if (pos_ < s_.size() && s_[pos_] == '}') {
      ++pos_;
      return n;
    }
    for (;;) {
      skip_blanks();
      const YamlNode key = make_scalar(take_token(":,}"), line_);
      if (pos_ >= s_.size() || s_[pos_] != ':') {
        fail(line_, "expected ':' in flow mapping");
      }
      ++pos_;
      n.entries.emplace_back(key.scalar, parse_value());
      skip_blanks();
      if (pos_ >= s_.size()) {
        fail(line_, "flow mapping must be closed on the same line");
      }
      if (s_[pos_] == ',') {
        ++pos_;
        continue;
      }
      if (s_[pos_] == '}') {
        ++pos_;
        return n;
      }
      fail(line_, "expected ',' or '}' in flow mapping");
    }
  }

  const std::string& s_;
  int line_;
  std::size_t pos_ = 0;
};

YamlNode parse_inline(const std::string& text, int line) {
  const std::string t = trim(text);
  if (!t.empty() && (t[0] == '[' || t[0] == '{')) {
    return FlowParser(t, line).parse_all();
  }
  return make_scalar(t, line);
}

class BlockParser {
 public:
  explicit BlockParser(std::vector<Line> lines) : lines_(std::move(lines)) {}

  YamlNode parse_document() {
    if (lines_.empty()) {
      return YamlNode{};
    }
    YamlNode root = parse_block(lines_[0].indent);
    if (pos_ != lines_.size()) {
      fail(lines_[pos_].number, "unexpected indentation");
    }
    return root;
  }

 private:
  static bool is_item(const std::string& t) { return t == "-" || (t.size() >= 2 && t[0] == '-' && t[1] == ' '); }

  YamlNode parse_block(int indent) {
    const Line& first = lines_[pos_];
    if (first.indent != indent) {
      fail(first.number, "unexpected indentation");
    }
    if (is_item(first.text)) {
      return parse_sequence(indent);
    }
    if (key_separator(first.text) != std::string::npos) {
      return parse_mapping(indent);
    }
    YamlNode n = parse_inline(first.text, first.number);
    ++pos_;
    return n;
  }

  YamlNode parse_sequence(int indent) {
    YamlNode seq;
    seq.kind = YamlNode::kSequence;
    seq.line = lines_[pos_].number;
    while (pos_ < lines_.size() && lines_[pos_].indent == indent && is_item(lines_[pos_].text)) {
      Line& cur = lines_[pos_];
      std::size_t skip = 1;
      while (skip < cur.text.size() && cur.text[skip] == ' ') {
        ++skip;
      }
      const std::string rest = cur.text.substr(skip);
      if (rest.empty()) {
        ++pos_;
        if (pos_ < lines_.size() && lines_[pos_].indent > indent) {
          seq.items.push_back(parse_block(lines_[pos_].indent));
        } else {
          seq.items.emplace_back();
        }
        continue;
      }
      // Re-read the remainder as a line that starts where its text starts.
      cur.indent = indent + static_cast<int>(skip);
      cur.text = rest;
      seq.items.push_back(parse_block(cur.indent));
    }
    if (pos_ < lines_.size() && lines_[pos_].indent > indent) {
      fail(lines_[pos_].number, "unexpected indentation");
    }
    return seq;
  }

  YamlNode parse_mapping(int indent) {
    YamlNode map;
    map.kind = YamlNode::kMapping;
    map.line = lines_[pos_].number;
    while (pos_ < lines_.size() && lines_[pos_].indent == indent) {
      const Line cur = lines_[pos_];
      if (is_item(cur.text)) {
        break;
      }
      const std::size_t sep = key_separator(cur.text);
      if (sep == std::string::npos) {
        fail(cur.number, "expected 'key: value'");
      }
      const YamlNode key = make_scalar(cur.text.substr(0, sep), cur.number);
      if (key.kind != YamlNode::kScalar) {
        fail(cur.number, "mapping key must be a scalar");
      }
      for (const auto& e : map.entries) {
        if (e.first == key.scalar) {
          fail(cur.number, "duplicate mapping key '" + key.scalar + "'");
        }
      }
      const std::string rest = trim(cur.text.substr(sep + 1));
      ++pos_;
      if (!rest.empty()) {
        map.entries.emplace_back(key.scalar, parse_inline(rest, cur.number));
        if (pos_ < lines_.size() && lines_[pos_].indent > indent) {
          fail(lines_[pos_].number, "unexpected indentation");
        }
      } else if (pos_ < lines_.size() && lines_[pos_].indent > indent) {
        map.entries.emplace_back(key.scalar, parse_block(lines_[pos_].indent));
      } else if (pos_ < lines_.size() && lines_[pos_].indent == indent && is_item(lines_[pos_].text)) {
        map.entries.emplace_back(key.scalar, parse_sequence(indent));  // "key:\n- a\n- b"
      } else {
        YamlNode null_node;
        null_node.line = cur.number;
        map.entries.emplace_back(key.scalar, null_node);
      }
    }
    return map;
  }

  std::vector<Line> lines_;
  std::size_t pos_ = 0;
};

}  // namespace

const YamlNode* YamlNode::find(const std::string& key) const {
  if (kind != kMapping) {
    return nullptr;
  }
  for (const auto& e : entries) {
    if (e.first == key) {
      return &e.second;
    }
  }
  return nullptr;
}

YamlNode parse_yaml(const std::string& text) { return BlockParser(split_lines(text)).parse_document(); }

YamlNode parse_yaml_file(const std::string& path) {
  std::ifstream in(path);
  if (!in) {
    throw std::runtime_error("cannot read " + path);
  }
  std::stringstream buf;
  buf << in.rdbuf();
  return parse_yaml(buf.str());
}

}  // namespace msharp
