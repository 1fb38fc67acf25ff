// Shared host-side types of the serving engine: return codes, Status, sampling configuration
// and its validation, small time helpers.
//
// Return-code values and the validation rules follow the reference so that clients see the same
// numbers (src/ksana_llm/utils/ret_code.h; src/ksana_llm/utils/request.h:22-62;
// src/ksana_llm/utils/request.cpp:12-30).
#pragma once
#include <chrono>
#include <cstdint>
#include <string>
#include <vector>

namespace ksana {

enum RetCode : int {
  RET_SUCCESS = 0,
  RET_INVALID_ARGUMENT = 1,
  RET_SEGMENT_FAULT = 2,
  RET_OUT_OF_MEMORY = 3,
  RET_TERMINATED = 4,
  RET_EXCEED_CAPACITY = 5,
  RET_EXCEED_LENGTH = 6,
  RET_TIMEOUT = 7,
  RET_ALLOCATE_FAIL = 8,
  RET_FREE_FAIL = 9,
  RET_UNDEFINED_REFERENCE = 10,
  RET_STOP_ITERATION = 11,
  RET_RUNTIME = 12,
  RET_UNKNOWN = 255,
};

struct Status {
  RetCode code = RET_SUCCESS;
  std::string message;
  Status() = default;
  Status(RetCode c, std::string m) : code(c), message(std::move(m)) {}
  bool ok() const { return code == RET_SUCCESS; }
};

struct SamplingConfig {
  int topk = 1;
  int num_beams = 1;
  int num_return_sequences = 1;
  float topp = 1.0f;
  float temperature = 1.0f;
  float repetition_penalty = 1.0f;
  float length_penalty = 1.0f;
  int no_repeat_ngram_size = 0;
  int encoder_no_repeat_ngram_size = 0;
  int max_new_tokens = 1024;
  int logprobs_num = 0;
  std::vector<int> stop_token_ids;
  std::vector<std::string> stop_strings;
  bool ignore_eos = false;
  uint64_t seed = 0;   // 0: engine picks one per request

  // topp / temperature of 0 mean "off" (1); topk must be in [1, 1024]; the two n-gram options
  // exclude each other; beams need as many log-probs as beams.
  Status VerifyArgs() {
    if (topp == 0.0f) topp = 1.0f;
    if (temperature == 0.0f) temperature = 1.0f;
    if (topp < 0.0f || topp > 1.0f) return Status(RET_INVALID_ARGUMENT, "topp must be in (0, 1]");
    if (temperature < 0.0f) return Status(RET_INVALID_ARGUMENT, "temperature must be positive");
    if (topk > 1024) return Status(RET_INVALID_ARGUMENT, "topk should not be larger than 1024");
    if (topk < 1) return Status(RET_INVALID_ARGUMENT, "topk should not be smaller than 1");
    if (no_repeat_ngram_size > 0 && encoder_no_repeat_ngram_size > 0)
      return Status(RET_INVALID_ARGUMENT,
                    "no_repeat_ngram_size and encoder_no_repeat_ngram_size cannot both be set");
    if (num_beams < 1 || num_return_sequences < 1)
      return Status(RET_INVALID_ARGUMENT, "num_beams and num_return_sequences must be >= 1");
    if (max_new_tokens < 0) return Status(RET_INVALID_ARGUMENT, "max_new_tokens must be >= 0");
    if (repetition_penalty <= 0.0f) return Status(RET_INVALID_ARGUMENT, "repetition_penalty must be positive");
    if (num_beams > 1 && logprobs_num < num_beams) logprobs_num = num_beams;
    return Status();
  }
};

inline int64_t NowMs() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch())
      .count();
}
inline int64_t NowUs() {
  return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

inline int CeilDiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace ksana
