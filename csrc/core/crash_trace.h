// Native stack of a crashing thread.
//
// A fault in one of the engine's own threads (sender pool, completion poller, server connections)
// kills the serving process with no trace of where: the interpreter's fault handler prints Python
// frames only, and those threads have none.  With BLLM_KVTRANS_CRASH_TRACE=1 the module installs a
// handler for SIGSEGV, SIGBUS, SIGFPE, SIGILL and SIGABRT that writes the faulting thread's native
// frames to stderr as `module(+0xoffset)` lines (resolvable with addr2line against the module, which
// is built with line tables), then hands the signal to whatever handler was installed before.
#pragma once

namespace kvx {

// Idempotent.  Returns true when the handlers are (already) installed.
bool install_crash_trace(bool force = false);

}  // namespace kvx
