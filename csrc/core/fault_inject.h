// Host-side fault injection for the transfer path.  The reference compiles its hooks only into
// debug builds (kvtransfer/src/fault_inject.cpp:12-35); here they are always present and off
// unless BLLM_KVTRANS_DEBUG_TX_FAILRATE > 1, and tests can also arm a deterministic countdown.
// Nothing here touches a GPU: injected failures are C++ exceptions and sleeps on host threads.
#pragma once
namespace kvx {
void fault_inject_throw();                 // throws std::runtime_error with probability (rate-1)%
void fault_inject_sleep(int max_us);       // sleeps up to max_us with the same probability
void fault_inject_arm(int throw_after_n);  // test hook: the n-th next call to fault_inject_throw throws (<=0 disarms)
}  // namespace kvx
