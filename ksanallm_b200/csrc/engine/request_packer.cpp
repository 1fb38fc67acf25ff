#include "request_packer.h"

#include <cstring>
#include <stdexcept>

#ifndef KSANA_NO_PYBIND
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#endif

namespace ksana {

const MsgValue* MsgValue::Find(const std::string& key) const {
  if (kind != MAP) return nullptr;
  for (const auto& kv : fields)
    if (kv.first.kind == STR && kv.first.s == key) return &kv.second;
  return nullptr;
}

namespace {

struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  int depth = 0;
  void Need(size_t n) const {
    if (static_cast<size_t>(end - p) < n) throw std::runtime_error("msgpack: truncated input");
  }
  uint64_t Be(int n) {
    Need(n);
    uint64_t v = 0;
    for (int k = 0; k < n; ++k) v = (v << 8) | *p++;
    return v;
  }
  std::string Bytes(size_t n) {
    Need(n);
    std::string s(reinterpret_cast<const char*>(p), n);
    p += n;
    return s;
  }
  MsgValue Array(size_t n) {
    MsgValue v;
    v.kind = MsgValue::ARRAY;
    Need(n);                                   // every element takes at least one byte
    v.items.reserve(n);
    for (size_t k = 0; k < n; ++k) v.items.push_back(Value());
    return v;
  }
  MsgValue Map(size_t n) {
    MsgValue v;
    v.kind = MsgValue::MAP;
    Need(2 * n);
    v.fields.reserve(n);
    for (size_t k = 0; k < n; ++k) {
      MsgValue key = Value();
      v.fields.emplace_back(std::move(key), Value());
    }
    return v;
  }
  MsgValue Value() {
    if (++depth > 64) throw std::runtime_error("msgpack: nesting too deep");
    Need(1);
    const uint8_t t = *p++;
    MsgValue v;
    if (t <= 0x7f) { v.kind = MsgValue::INT; v.i = t; }
    else if (t >= 0xe0) { v.kind = MsgValue::INT; v.i = static_cast<int8_t>(t); }
    else if ((t & 0xf0) == 0x80) v = Map(t & 0x0f);
    else if ((t & 0xf0) == 0x90) v = Array(t & 0x0f);
    else if ((t & 0xe0) == 0xa0) { v.kind = MsgValue::STR; v.s = Bytes(t & 0x1f); }
    else switch (t) {
      case 0xc0: break;
      case 0xc2: v.kind = MsgValue::BOOL; v.b = false; break;
      case 0xc3: v.kind = MsgValue::BOOL; v.b = true; break;
      case 0xc4: v.kind = MsgValue::BIN; v.s = Bytes(Be(1)); break;
      case 0xc5: v.kind = MsgValue::BIN; v.s = Bytes(Be(2)); break;
      case 0xc6: v.kind = MsgValue::BIN; v.s = Bytes(Be(4)); break;
      case 0xca: { uint32_t raw = static_cast<uint32_t>(Be(4)); float f; std::memcpy(&f, &raw, 4); v.kind = MsgValue::FLOAT; v.f = f; break; }
      case 0xcb: { uint64_t raw = Be(8); std::memcpy(&v.f, &raw, 8); v.kind = MsgValue::FLOAT; break; }
      case 0xcc: v.kind = MsgValue::INT; v.i = static_cast<int64_t>(Be(1)); break;
      case 0xcd: v.kind = MsgValue::INT; v.i = static_cast<int64_t>(Be(2)); break;
      case 0xce: v.kind = MsgValue::INT; v.i = static_cast<int64_t>(Be(4)); break;
      case 0xcf: { v.u = Be(8); if (v.u <= INT64_MAX) { v.kind = MsgValue::INT; v.i = static_cast<int64_t>(v.u); } else v.kind = MsgValue::UINT; break; }
      case 0xd0: v.kind = MsgValue::INT; v.i = static_cast<int8_t>(Be(1)); break;
      case 0xd1: v.kind = MsgValue::INT; v.i = static_cast<int16_t>(Be(2)); break;
      case 0xd2: v.kind = MsgValue::INT; v.i = static_cast<int32_t>(Be(4)); break;
      case 0xd3: v.kind = MsgValue::INT; v.i = static_cast<int64_t>(Be(8)); break;
      case 0xd9: v.kind = MsgValue::STR; v.s = Bytes(Be(1)); break;
      case 0xda: v.kind = MsgValue::STR; v.s = Bytes(Be(2)); break;
      case 0xdb: v.kind = MsgValue::STR; v.s = Bytes(Be(4)); break;
      case 0xdc: v = Array(Be(2)); break;
      case 0xdd: v = Array(Be(4)); break;
      case 0xde: v = Map(Be(2)); break;
      case 0xdf: v = Map(Be(4)); break;
      default: throw std::runtime_error("msgpack: unsupported type byte (extension types are not part of this protocol)");
    }
    --depth;
    return v;
  }
};

void PutBe(std::string* out, uint64_t v, int n) {
  for (int k = n - 1; k >= 0; --k) out->push_back(static_cast<char>((v >> (8 * k)) & 0xff));
}

void Write(const MsgValue& v, std::string* out) {
  switch (v.kind) {
    case MsgValue::NIL: out->push_back(static_cast<char>(0xc0)); break;
    case MsgValue::BOOL: out->push_back(static_cast<char>(v.b ? 0xc3 : 0xc2)); break;
    case MsgValue::UINT: out->push_back(static_cast<char>(0xcf)); PutBe(out, v.u, 8); break;
    case MsgValue::INT: {
      const int64_t i = v.i;
      if (i >= 0) {
        if (i <= 0x7f) out->push_back(static_cast<char>(i));
        else if (i <= 0xff) { out->push_back(static_cast<char>(0xcc)); PutBe(out, i, 1); }
        else if (i <= 0xffff) { out->push_back(static_cast<char>(0xcd)); PutBe(out, i, 2); }
        else if (i <= 0xffffffffLL) { out->push_back(static_cast<char>(0xce)); PutBe(out, i, 4); }
        else { out->push_back(static_cast<char>(0xcf)); PutBe(out, i, 8); }
      } else {
        if (i >= -32) out->push_back(static_cast<char>(i));
        else if (i >= INT8_MIN) { out->push_back(static_cast<char>(0xd0)); PutBe(out, static_cast<uint8_t>(i), 1); }
        else if (i >= INT16_MIN) { out->push_back(static_cast<char>(0xd1)); PutBe(out, static_cast<uint16_t>(i), 2); }
        else if (i >= INT32_MIN) { out->push_back(static_cast<char>(0xd2)); PutBe(out, static_cast<uint32_t>(i), 4); }
        else { out->push_back(static_cast<char>(0xd3)); PutBe(out, static_cast<uint64_t>(i), 8); }
      }
      break;
    }
    case MsgValue::FLOAT: { uint64_t raw; std::memcpy(&raw, &v.f, 8); out->push_back(static_cast<char>(0xcb)); PutBe(out, raw, 8); break; }
    case MsgValue::STR: {
      const size_t n = v.s.size();
      if (n <= 31) out->push_back(static_cast<char>(0xa0 | n));
      else if (n <= 0xff) { out->push_back(static_cast<char>(0xd9)); PutBe(out, n, 1); }
      else if (n <= 0xffff) { out->push_back(static_cast<char>(0xda)); PutBe(out, n, 2); }
      else { out->push_back(static_cast<char>(0xdb)); PutBe(out, n, 4); }
      out->append(v.s);
      break;
    }
    case MsgValue::BIN: {
      const size_t n = v.s.size();
      if (n <= 0xff) { out->push_back(static_cast<char>(0xc4)); PutBe(out, n, 1); }
      else if (n <= 0xffff) { out->push_back(static_cast<char>(0xc5)); PutBe(out, n, 2); }
      else { out->push_back(static_cast<char>(0xc6)); PutBe(out, n, 4); }
      out->append(v.s);
      break;
    }
    case MsgValue::ARRAY: {
      const size_t n = v.items.size();
      if (n <= 15) out->push_back(static_cast<char>(0x90 | n));
      else if (n <= 0xffff) { out->push_back(static_cast<char>(0xdc)); PutBe(out, n, 2); }
      else { out->push_back(static_cast<char>(0xdd)); PutBe(out, n, 4); }
      for (const auto& it : v.items) Write(it, out);
      break;
    }
    case MsgValue::MAP: {
      const size_t n = v.fields.size();
      if (n <= 15) out->push_back(static_cast<char>(0x80 | n));
      else if (n <= 0xffff) { out->push_back(static_cast<char>(0xde)); PutBe(out, n, 2); }
      else { out->push_back(static_cast<char>(0xdf)); PutBe(out, n, 4); }
      for (const auto& kv : v.fields) { Write(kv.first, out); Write(kv.second, out); }
      break;
    }
  }
}

bool IsIntArray(const MsgValue* v) {
  if (!v || v->kind != MsgValue::ARRAY) return false;
  for (const auto& it : v->items)
    if (it.kind != MsgValue::INT) return false;
  return true;
}

}  // namespace

MsgValue MsgUnpack(const std::string& bytes) {
  Reader r{reinterpret_cast<const uint8_t*>(bytes.data()), reinterpret_cast<const uint8_t*>(bytes.data()) + bytes.size()};
  MsgValue v = r.Value();
  if (r.p != r.end) throw std::runtime_error("msgpack: trailing bytes after the document");
  return v;
}

std::string MsgPack(const MsgValue& v) {
  std::string out;
  Write(v, &out);
  return out;
}

std::string ValidateForwardBody(const MsgValue& doc) {
  const MsgValue* reqs = doc.Find("requests");
  if (!reqs || reqs->kind != MsgValue::ARRAY || reqs->items.empty()) return "no requests";
  for (const MsgValue& r : reqs->items) {
    if (r.kind != MsgValue::MAP) return "a request is not a map";
    const MsgValue* tokens = r.Find("input_tokens");
    const MsgValue* prompt = r.Find("prompt");
    const bool has_tokens = tokens && tokens->kind == MsgValue::ARRAY && !tokens->items.empty();
    if (has_tokens && !IsIntArray(tokens)) return "input_tokens must be integers";
    if (!has_tokens && !(prompt && prompt->kind == MsgValue::STR)) return "request needs input_tokens or a prompt";
    const MsgValue* targets = r.Find("request_target");
    if (!targets || targets->kind != MsgValue::ARRAY || targets->items.empty()) return "request_target is empty";
    for (const MsgValue& t : targets->items) {
      const MsgValue* name = t.Find("target_name");
      if (!name || name->kind != MsgValue::STR) return "request_target entry without target_name";
      if (name->s != "layernorm" && name->s != "transformer" && name->s != "logits")
        return "unknown target_name " + name->s;
      const MsgValue* ids = t.Find("token_id");
      if (ids && ids->kind != MsgValue::NIL && !IsIntArray(ids)) return "token_id must be integers";
      const MsgValue* mode = t.Find("token_reduce_mode");
      if (mode && mode->kind == MsgValue::STR && mode->s != "GATHER_ALL" && mode->s != "GATHER_TOKEN_ID")
        return "unknown token_reduce_mode " + mode->s;
      const MsgValue* slices = t.Find("slice_pos");
      if (slices && slices->kind == MsgValue::ARRAY)
        for (const MsgValue& p : slices->items)
          if (!IsIntArray(&p) || p.items.size() != 2) return "slice_pos entries must be [begin, end]";
    }
  }
  return "";
}

#ifndef KSANA_NO_PYBIND
namespace py = pybind11;

static py::object ToPy(const MsgValue& v) {
  switch (v.kind) {
    case MsgValue::NIL: return py::none();
    case MsgValue::BOOL: return py::bool_(v.b);
    case MsgValue::INT: return py::int_(v.i);
    case MsgValue::UINT: return py::int_(v.u);
    case MsgValue::FLOAT: return py::float_(v.f);
    case MsgValue::STR: return py::str(v.s);
    case MsgValue::BIN: return py::bytes(v.s);
    case MsgValue::ARRAY: {
      py::list l;
      for (const auto& it : v.items) l.append(ToPy(it));
      return std::move(l);
    }
    case MsgValue::MAP: {
      py::dict d;
      for (const auto& kv : v.fields) d[ToPy(kv.first)] = ToPy(kv.second);
      return std::move(d);
    }
  }
  return py::none();
}

static MsgValue FromPy(const py::handle& o) {
  MsgValue v;
  if (o.is_none()) return v;
  if (py::isinstance<py::bool_>(o)) { v.kind = MsgValue::BOOL; v.b = o.cast<bool>(); }
  else if (py::isinstance<py::int_>(o)) {
    try { v.kind = MsgValue::INT; v.i = o.cast<int64_t>(); }
    catch (const py::cast_error&) { v.kind = MsgValue::UINT; v.u = o.cast<uint64_t>(); }
  }
  else if (py::isinstance<py::float_>(o)) { v.kind = MsgValue::FLOAT; v.f = o.cast<double>(); }
  else if (py::isinstance<py::str>(o)) { v.kind = MsgValue::STR; v.s = o.cast<std::string>(); }
  else if (py::isinstance<py::bytes>(o) || py::isinstance<py::bytearray>(o)) { v.kind = MsgValue::BIN; v.s = py::bytes(py::reinterpret_borrow<py::object>(o)).cast<std::string>(); }
  else if (py::isinstance<py::dict>(o)) {
    v.kind = MsgValue::MAP;
    for (auto kv : py::reinterpret_borrow<py::dict>(o)) v.fields.emplace_back(FromPy(kv.first), FromPy(kv.second));
  }
  else if (py::isinstance<py::list>(o) || py::isinstance<py::tuple>(o)) {
    v.kind = MsgValue::ARRAY;
    for (auto it : py::reinterpret_borrow<py::sequence>(o)) v.items.push_back(FromPy(it));
  }
  else throw std::runtime_error("msgpack: cannot encode object of type " + std::string(py::str(py::type::of(o))));
  return v;
}

void BindRequestPacker(py::module_& m) {
  m.def("msgpack_unpack", [](const py::bytes& b) { return ToPy(MsgUnpack(b.cast<std::string>())); },
        "Decode a msgpack document into Python objects (strings as str, binaries as bytes).");
  m.def("msgpack_pack", [](const py::object& o) { return py::bytes(MsgPack(FromPy(o))); },
        "Encode Python objects (None, bool, int, float, str, bytes, list / tuple, dict) as msgpack.");
  m.def("unpack_forward_body", [](const py::bytes& b) {
    MsgValue doc = MsgUnpack(b.cast<std::string>());
    const std::string why = ValidateForwardBody(doc);
    if (!why.empty()) throw py::value_error(why);
    return ToPy(doc);
  }, "Decode and validate a /forward request body.");
}
#endif

}  // namespace ksana
