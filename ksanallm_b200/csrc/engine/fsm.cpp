#include "fsm.h"

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

namespace ksana {

namespace {

bool IsQuantifier(char c) { return c == '*' || c == '+' || c == '?' || c == '{'; }

// Length of the atom starting at p[i] when that atom is not a plain literal (class, group, dot,
// escape class). Returns 0 for a plain literal.
size_t NonLiteralAtomLen(const std::string& p, size_t i) {
  const char c = p[i];
  if (c == '.') return 1;
  if (c == '[') {
    size_t j = i + 1;
    if (j < p.size() && p[j] == '^') ++j;
    if (j < p.size() && p[j] == ']') ++j;
    while (j < p.size() && p[j] != ']') j += (p[j] == '\\' && j + 1 < p.size()) ? 2 : 1;
    return j < p.size() ? j - i + 1 : p.size() - i;
  }
  if (c == '(') {
    int depth = 0;
    size_t j = i;
    for (; j < p.size(); ++j) {
      if (p[j] == '\\') { ++j; continue; }
      if (p[j] == '[') { j += NonLiteralAtomLen(p, j) - 1; continue; }
      if (p[j] == '(') ++depth;
      if (p[j] == ')' && --depth == 0) break;
    }
    return j < p.size() ? j - i + 1 : p.size() - i;
  }
  if (c == '\\' && i + 1 < p.size()) {
    const char e = p[i + 1];
    if (e == 'd' || e == 'D' || e == 'w' || e == 'W' || e == 's' || e == 'S' || e == 'b' || e == 'B') return 2;
  }
  return 0;
}

size_t QuantifierLen(const std::string& p, size_t i) {
  if (i >= p.size() || !IsQuantifier(p[i])) return 0;
  size_t n = 1;
  if (p[i] == '{') {
    size_t j = p.find('}', i);
    n = j == std::string::npos ? p.size() - i : j - i + 1;
  }
  if (i + n < p.size() && p[i + n] == '?') ++n;   // lazy marker
  return n;
}

char Unescape(char e) {
  switch (e) {
    case 'n': return '\n';
    case 't': return '\t';
    case 'r': return '\r';
    case 'f': return '\f';
    case 'v': return '\v';
    default: return e;
  }
}

bool HasTopLevelAlternation(const std::string& p) {
  int depth = 0;
  for (size_t i = 0; i < p.size(); ++i) {
    if (p[i] == '\\') { ++i; continue; }
    if (p[i] == '[') { i += NonLiteralAtomLen(p, i) - 1; continue; }
    if (p[i] == '(') ++depth;
    if (p[i] == ')') --depth;
    if (p[i] == '|' && depth == 0) return true;
  }
  return false;
}

}  // namespace

FiniteStateMachine::FiniteStateMachine(const std::string& pattern) {
  auto push_gen = [&](const std::string& sub) {
    if (!segments_.empty() && segments_.back().type == FsmSegmentType::GENERATION) segments_.back().text += sub;
    else segments_.push_back({FsmSegmentType::GENERATION, sub});
  };
  auto push_const = [&](char c) {
    if (!segments_.empty() && segments_.back().type == FsmSegmentType::CONSTANT) segments_.back().text.push_back(c);
    else segments_.push_back({FsmSegmentType::CONSTANT, std::string(1, c)});
  };
  std::string p = pattern;
  if (!p.empty() && p.front() == '^') p.erase(0, 1);
  if (!p.empty() && p.back() == '$' && (p.size() < 2 || p[p.size() - 2] != '\\')) p.pop_back();
  if (HasTopLevelAlternation(p)) {
    push_gen(p);   // nothing is constant across alternatives
  } else {
    size_t i = 0;
    while (i < p.size()) {
      size_t alen = NonLiteralAtomLen(p, i);
      if (alen > 0) {
        const size_t q = QuantifierLen(p, i + alen);
        push_gen(p.substr(i, alen + q));
        i += alen + q;
        continue;
      }
      // plain literal (possibly escaped)
      size_t llen = 1;
      char lit = p[i];
      if (p[i] == '\\' && i + 1 < p.size()) { lit = Unescape(p[i + 1]); llen = 2; }
      const size_t q = QuantifierLen(p, i + llen);
      if (q > 0) {
        push_gen(p.substr(i, llen + q));   // a repeated literal is not constant text
      } else {
        push_const(lit);
      }
      i += llen + q;
    }
  }
  for (auto& s : segments_) {
    if (s.type != FsmSegmentType::GENERATION) continue;
    try {
      s.re = std::regex(s.text, std::regex::ECMAScript);
      s.has_regex = true;
    } catch (const std::regex_error&) {
      s.has_regex = false;   // unsupported syntax: the segment ends at the next constant's first character
    }
  }
}

FsmStepResult FiniteStateMachine::Step(const std::string& generated, int segment, size_t segment_start) const {
  FsmStepResult r;
  r.text = generated;
  r.segment = segment;
  r.segment_start = std::min(segment_start, generated.size());
  const int n = static_cast<int>(segments_.size());
  while (r.segment < n) {
    const FsmSegment& seg = segments_[r.segment];
    if (seg.type == FsmSegmentType::CONSTANT) {
      // inject the constant (whatever was sampled past the segment start is replaced)
      std::string next = r.text.substr(0, r.segment_start) + seg.text;
      if (next != r.text) { r.text = std::move(next); r.changed = true; }
      r.segment_start = r.text.size();
      ++r.segment;
      continue;
    }
    // generation segment: look for the point where the following constant begins
    if (r.segment + 1 >= n) break;   // trailing free segment: runs until EOS / length limits
    const char first = segments_[r.segment + 1].text[0];
    const std::string g = r.text.substr(r.segment_start);
    size_t cut = std::string::npos;
    for (size_t p = g.find(first); p != std::string::npos; p = g.find(first, p + 1)) {
      if (!seg.has_regex || std::regex_match(g.substr(0, p), seg.re)) { cut = p; break; }
    }
    if (cut == std::string::npos) break;
    if (r.segment_start + cut != r.text.size()) r.changed = true;
    r.text = r.text.substr(0, r.segment_start + cut);
    r.segment_start = r.text.size();
    ++r.segment;
  }
  r.final_state = r.segment >= n;
  return r;
}

std::shared_ptr<FiniteStateMachine> FsmController::GetOrCreate(const std::string& pattern) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = cache_.find(pattern);
  if (it != cache_.end()) return it->second;
  auto fsm = std::make_shared<FiniteStateMachine>(pattern);
  cache_[pattern] = fsm;
  return fsm;
}

size_t FsmController::size() {
  std::lock_guard<std::mutex> g(mu_);
  return cache_.size();
}

void BindFsm(pybind11::module_& m) {
  namespace py = pybind11;
  py::class_<FiniteStateMachine, std::shared_ptr<FiniteStateMachine>>(m, "FiniteStateMachine")
      .def(py::init<const std::string&>())
      .def("segments", [](const FiniteStateMachine& f) {
        std::vector<std::pair<int, std::string>> out;
        for (auto& s : f.segments()) out.emplace_back(static_cast<int>(s.type), s.text);
        return out;
      })
      .def("step", [](const FiniteStateMachine& f, const std::string& text, int segment, size_t start) {
        FsmStepResult r = f.Step(text, segment, start);
        return py::make_tuple(r.changed, r.final_state, r.text, r.segment, r.segment_start);
      });
  py::class_<FsmController>(m, "FsmController")
      .def(py::init<>())
      .def("get_or_create", &FsmController::GetOrCreate)
      .def("size", &FsmController::size);
}

}  // namespace ksana
