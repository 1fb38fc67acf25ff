// Structured output by "jump-forward" decoding: a regular expression is compiled into a chain of
// segments - constant text that is injected without sampling, and free segments that are sampled
// until the first character of the following constant appears - ending in a final state.
// This is not logit masking. Observable behaviour follows the reference
// (src/ksana_llm/utils/finite_state_machine.cpp:153-493 and
//  src/ksana_llm/batch_scheduler/strategy/continuous_batching.cpp:57-138); the compiler here is an
// own small regex splitter, so no regex library beyond <regex> is needed.
#pragma once
#include <memory>
#include <mutex>
#include <regex>
#include <string>
#include <unordered_map>
#include <vector>

namespace pybind11 { class module_; }

namespace ksana {

enum class FsmSegmentType : int { CONSTANT = 0, GENERATION = 1 };

struct FsmSegment {
  FsmSegmentType type;
  std::string text;      // constant text, or the sub-pattern of a generation segment
  bool has_regex = false;
  std::regex re;         // compiled sub-pattern (generation segments)
};

struct FsmStepResult {
  bool changed = false;  // `text` differs from the input: re-tokenise and replace the generated tokens
  bool final_state = false;
  std::string text;
  int segment = 0;       // cursor after the step
  size_t segment_start = 0;
};

class FiniteStateMachine {
 public:
  explicit FiniteStateMachine(const std::string& pattern);
  const std::vector<FsmSegment>& segments() const { return segments_; }
  // Advance from cursor (segment, segment_start) given everything generated so far.
  FsmStepResult Step(const std::string& generated, int segment, size_t segment_start) const;

 private:
  std::vector<FsmSegment> segments_;
};

// One compiled machine per pattern string, shared by all requests.
class FsmController {
 public:
  std::shared_ptr<FiniteStateMachine> GetOrCreate(const std::string& pattern);
  size_t size();

 private:
  std::mutex mu_;
  std::unordered_map<std::string, std::shared_ptr<FiniteStateMachine>> cache_;
};

void BindFsm(pybind11::module_& m);

}  // namespace ksana
