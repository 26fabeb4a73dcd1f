// Where the host time of a device collective goes (HOROVOD_HOST_TRACE=1):
// the executing thread drops named marks between the start of a response and
// its last launch; the time since the previous mark is added up per
// (response type, mark) and printed when the executor shuts down. Off by
// default; a mark then costs one predictable branch.
#ifndef HVD_B200_HOST_TRACE_H
#define HVD_B200_HOST_TRACE_H

namespace hvd {
namespace host_trace {

bool Enabled();
// Starts the clock for a response of the given type (Response::Type).
void Begin(int type);
// Adds the time since the previous mark (or Begin) under `label`.
void Mark(const char* label);
// Prints the averages to stderr and clears them.
void Report(int rank);

}  // namespace host_trace
}  // namespace hvd

#endif
