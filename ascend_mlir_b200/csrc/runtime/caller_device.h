// The calling thread's current CUDA device, kept across a call of this library.
//
// Every entry point that does device work makes its executor's (or mailbox's) device current.  A host program
// that shares the thread with other CUDA users (a framework whose allocator follows the current device) must
// find its own device current again afterwards: otherwise its next allocation lands on this library's device
// and a kernel on the first device reads memory it has no mapping for.  CallerDeviceScope remembers the
// device at construction and puts it back at destruction if the call changed it.  A thread that has no current
// context yet is left alone (making "device 0" current for it would create a context there).
#pragma once

namespace afir {

class CallerDeviceScope {
public:
  CallerDeviceScope();
  ~CallerDeviceScope();
  CallerDeviceScope(const CallerDeviceScope &) = delete;
  CallerDeviceScope &operator=(const CallerDeviceScope &) = delete;

private:
  int previous_ = -1;
};

} // namespace afir
