// Minimal JSON text writer. Numbers are streamed with default ostream formatting, which is
// what the reference's report does (src/main.cc:295-354); strings use the same escape set
// as src/runtime.cc:357-382 plus \u00XX for the remaining control characters.
#pragma once

#include <cstdint>
#include <sstream>
#include <string>
#include <vector>

namespace msharp {

std::string json_escape(const std::string& value);

class JsonWriter {
 public:
  JsonWriter& begin_object();
  JsonWriter& end_object();
  JsonWriter& begin_array();
  JsonWriter& end_array();
  JsonWriter& key(const std::string& name);
  JsonWriter& value(const std::string& v);
  JsonWriter& value(const char* v);
  JsonWriter& value(bool v);
  JsonWriter& value(int v);
  JsonWriter& value(int64_t v);
  JsonWriter& value(uint64_t v);
  JsonWriter& value(double v);
  JsonWriter& value(float v);
  JsonWriter& null();
  JsonWriter& raw(const std::string& json_text);  // pre-serialised value
  std::string str() const { return os_.str(); }

 private:
  void separator();
  std::ostringstream os_;
  std::vector<bool> first_;  // one flag per open container: no element written yet
  bool after_key_ = false;
};

}  // namespace msharp
