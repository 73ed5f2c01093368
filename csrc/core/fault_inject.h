// Host-side fault injection for the transfer path.  The reference compiles its hooks only into
// debug builds (kvtransfer/src/fault_inject.cpp:12-35); here they are always present and off
// unless BLLM_KVTRANS_DEBUG_TX_FAILRATE > 1, and tests can also arm a deterministic countdown.
// Nothing here touches a GPU: injected failures are C++ exceptions and sleeps on host threads.
#pragma once
namespace kvx {
void fault_inject_throw();                 // throws std::runtime_error with probability (rate-1)%
void fault_inject_sleep(int max_us);       // sleeps up to max_us with the same probability
void fault_inject_arm(int throw_after_n);  // test hook: the n-th next call to fault_inject_throw throws (<=0 disarms)
// Test hook for the asynchronous completion path: the next n batches of a device transport enqueue no
// completion record, so their completion never arrives and the poller's deadline has to fail them.  The
// GPU is not involved: the kernels of the batch run and finish as usual, only the record is left out.
void fault_inject_arm_drop_completion(int n);
bool fault_inject_drop_completion();
// Test hook for the end-to-end transfer check: the sender's next n checks perturb their own sum, so the
// comparison with the destination's sum fails although the data is intact.
void fault_inject_arm_corrupt_check(int n);
bool fault_inject_corrupt_check();
}  // namespace kvx
