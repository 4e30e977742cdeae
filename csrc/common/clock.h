// Wall-clock helpers (reference: include/common/time.h:8-10): the launch stamp names the log
// file, nanosecond stamps go into control-plane messages and traces.
#pragma once
#include <cstdint>
#include <string>

namespace pccl {
const std::string& launchTimestamp();   // "HH-MM-SS.uuuuuu" taken at library load
uint64_t nowNanos();                    // system clock, ns since epoch
uint64_t monotonicNanos();              // steady clock, for intervals
std::string nowString();                // "YYYY-MM-DD HH:MM:SS.uuuuuu"
}  // namespace pccl
