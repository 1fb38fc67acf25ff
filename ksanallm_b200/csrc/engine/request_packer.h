// msgpack wire format of the /forward endpoint, decoded and encoded natively
// (src/ksana_llm/utils/request_packer.cpp:1-124, request_serial.h:15-66 in the reference use msgpack-c).
// A small value tree (nil, bool, int, float, string, binary, array, map with string keys preserved in order) plus a
// strict decoder / encoder for the msgpack subset the endpoint exchanges; the pybind layer converts the tree to
// and from Python objects. Forward requests are validated here (token ids present, non-empty request targets,
// known reduce modes, well-formed slice positions) so that malformed bodies never reach the engine.
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

namespace pybind11 { class module_; }

namespace ksana {

struct MsgValue {
  enum Kind { NIL, BOOL, INT, UINT, FLOAT, STR, BIN, ARRAY, MAP } kind = NIL;
  bool b = false;
  int64_t i = 0;
  uint64_t u = 0;
  double f = 0.0;
  std::string s;                                        // STR and BIN payload
  std::vector<MsgValue> items;                          // ARRAY
  std::vector<std::pair<MsgValue, MsgValue>> fields;    // MAP in wire order
  const MsgValue* Find(const std::string& key) const;   // MAP lookup by string key (nullptr when absent)
};

// Throws std::runtime_error on truncated / unsupported input or trailing bytes.
MsgValue MsgUnpack(const std::string& bytes);
std::string MsgPack(const MsgValue& v);

// Checks a decoded /forward body; returns an empty string when it is acceptable, else the reason.
std::string ValidateForwardBody(const MsgValue& doc);

void BindRequestPacker(pybind11::module_& m);

}  // namespace ksana
