#include "msharp/json.h"

#include <cmath>
#include <cstdio>

namespace msharp {

std::string json_escape(const std::string& value) {
  std::string out;
  out.reserve(value.size() + 2);
  for (const char c : value) {
    switch (c) {
      case '\\':
        out += "\\\\";
        break;
      case '"':
        out += "\\\"";
        break;
      case '\n':
        out += "\\n";
        break;
      case '\r':
        out += "\\r";
        break;
      case '\t':
        out += "\\t";
        break;
      default:
        if (static_cast<unsigned char>(c) < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof(buf), "\\u%04x", static_cast<unsigned>(static_cast<unsigned char>(c)));
          out += buf;
        } else {
          out += c;
        }
    }
  }
  return out;
}

void JsonWriter::separator() {
  if (after_key_) {
    after_key_ = false;
    return;
  }
  if (!first_.empty()) {
    if (!first_.back()) {
      os_ << ",";
    }
    first_.back() = false;
  }
}

JsonWriter& JsonWriter::begin_object() {
  separator();
  os_ << "{";
  first_.push_back(true);
  return *this;
}

JsonWriter& JsonWriter::end_object() {
  os_ << "}";
  first_.pop_back();
  return *this;
}

JsonWriter& JsonWriter::begin_array() {
  separator();
  os_ << "[";
  first_.push_back(true);
  return *this;
}

JsonWriter& JsonWriter::end_array() {
  os_ << "]";
  first_.pop_back();
  return *this;
}

JsonWriter& JsonWriter::key(const std::string& name) {
  separator();
  os_ << "\"" << json_escape(name) << "\":";
  after_key_ = true;
  return *this;
}

JsonWriter& JsonWriter::value(const std::string& v) {
  separator();
  os_ << "\"" << json_escape(v) << "\"";
  return *this;
}

JsonWriter& JsonWriter::value(const char* v) { return value(std::string(v)); }

JsonWriter& JsonWriter::value(bool v) {
  separator();
  os_ << (v ? "true" : "false");
  return *this;
}

JsonWriter& JsonWriter::value(int v) {
  separator();
  os_ << v;
  return *this;
}

JsonWriter& JsonWriter::value(int64_t v) {
  separator();
  os_ << v;
  return *this;
}

JsonWriter& JsonWriter::value(uint64_t v) {
  separator();
  os_ << v;
  return *this;
}

JsonWriter& JsonWriter::value(double v) {
  separator();
  if (std::isfinite(v)) {
    os_ << v;
  } else {
    os_ << "null";  // JSON has no NaN / infinity
  }
  return *this;
}

JsonWriter& JsonWriter::value(float v) { return value(static_cast<double>(v)); }

JsonWriter& JsonWriter::null() {
  separator();
  os_ << "null";
  return *this;
}

JsonWriter& JsonWriter::raw(const std::string& json_text) {
  separator();
  os_ << json_text;
  return *this;
}

}  // namespace msharp
