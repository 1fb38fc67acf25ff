#include "stop_checker.h"

#include <algorithm>

#ifndef KSANA_NO_PYBIND
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#endif

namespace ksana {

StopChecker::StopChecker(std::vector<std::string> stops) {
  for (auto& s : stops) {
    if (s.empty()) continue;                 // an empty stop string would match everywhere
    max_stop_ = std::max(max_stop_, s.size());
    stops_.push_back(std::move(s));
  }
}

bool StopChecker::EndsIncomplete(const std::string& piece) {
  const size_t n = piece.size();
  if (n >= 3 && static_cast<unsigned char>(piece[n - 3]) == 0xEF && static_cast<unsigned char>(piece[n - 2]) == 0xBF &&
      static_cast<unsigned char>(piece[n - 1]) == 0xBD)
    return true;                             // U+FFFD: the detokeniser saw half a character
  // a lead byte without all of its continuation bytes at the very end
  for (size_t back = 1; back <= 3 && back <= n; ++back) {
    const unsigned char c = static_cast<unsigned char>(piece[n - back]);
    if ((c & 0xC0) == 0x80) continue;        // continuation byte: keep looking for its lead
    if (c < 0x80) return false;
    const size_t need = (c & 0xE0) == 0xC0 ? 2 : ((c & 0xF0) == 0xE0 ? 3 : ((c & 0xF8) == 0xF0 ? 4 : 1));
    return back < need;
  }
  return false;
}

long StopChecker::Append(const std::string& piece) {
  if (hit_ >= 0) return hit_;
  const size_t old = text_.size();
  text_ += piece;
  if (stops_.empty() || piece.empty()) return -1;
  // a match that uses the new piece starts no earlier than max_stop - 1 bytes before it
  const size_t from = old >= max_stop_ - 1 ? old - (max_stop_ - 1) : 0;
  size_t best = std::string::npos;
  for (const auto& s : stops_) {
    const size_t pos = text_.find(s, from);
    if (pos != std::string::npos && pos < best) best = pos;
  }
  if (best != std::string::npos) hit_ = static_cast<long>(best);
  return hit_;
}

std::string StopChecker::Kept() const { return hit_ >= 0 ? text_.substr(0, static_cast<size_t>(hit_)) : text_; }

void StopChecker::Reset() {
  text_.clear();
  hit_ = -1;
}

#ifndef KSANA_NO_PYBIND
void BindStopChecker(pybind11::module_& m) {
  namespace py = pybind11;
  py::class_<StopChecker>(m, "StopChecker")
      .def(py::init<std::vector<std::string>>())
      .def_static("ends_incomplete", [](const std::string& s) { return StopChecker::EndsIncomplete(s); })
      .def("append", &StopChecker::Append)
      .def("text", &StopChecker::text)
      .def("kept", &StopChecker::Kept)
      .def("reset", &StopChecker::Reset);
}
#endif

}  // namespace ksana
