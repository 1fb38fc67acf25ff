// Index guards: kernels that consume indices produced elsewhere (block tables, cache slots, positions, expert ids,
// destination rows) verify them before the access; a bad index is recorded once in the per-device error word as
// code * 1000000 + (value mod 1000000) and the access is skipped, so a bookkeeping bug shows up as a Python error
// with the offending value instead of an out-of-range device access.
#pragma once
namespace ksana {
enum GuardCode : int { kGuardBlockId = 11, kGuardQueryRow = 12, kGuardPosition = 13, kGuardSlot = 14, kGuardExpert = 15,
                       kGuardDstRow = 16, kGuardGatherRow = 17 };
__device__ __forceinline__ void guard_report(int* err, int code, long long value) {
  if (err) atomicCAS(err, 0, code * 1000000 + static_cast<int>((value < 0 ? -value : value) % 1000000));
}
}  // namespace ksana
