// Stop-string detection over incrementally decoded text
// (src/ksana_llm/utils/stop_checker.cpp:8-56 in the reference decodes the last token, strips a trailing U+FFFD,
// searches the stop strings and truncates the output). Here the detokeniser stays in Python (as the reference's
// tokenizer bridge does); this class owns the text of one output: pieces are appended as tokens arrive, a piece
// that ends inside a multi-byte character is held back, and only the tail that a new piece can complete is
// searched, so a generation of n tokens costs O(n) instead of a full re-decode and re-search per token.
#pragma once
#include <string>
#include <vector>

namespace pybind11 { class module_; }

namespace ksana {

class StopChecker {
 public:
  explicit StopChecker(std::vector<std::string> stops);
  // True when `piece` ends with U+FFFD or inside a UTF-8 sequence: the caller waits for more tokens.
  static bool EndsIncomplete(const std::string& piece);
  // Appends a decoded piece. Returns the byte offset in text() where the earliest stop string starts, or -1.
  long Append(const std::string& piece);
  const std::string& text() const { return text_; }
  // text() cut before the stop string found by the last Append (whole text when none was found)
  std::string Kept() const;
  void Reset();

 private:
  std::vector<std::string> stops_;
  size_t max_stop_ = 0;
  std::string text_;
  long hit_ = -1;
};

void BindStopChecker(pybind11::module_& m);

}  // namespace ksana
