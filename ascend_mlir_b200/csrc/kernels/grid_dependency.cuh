// Programmatic dependent launch, device side (also compiled at run time as a header of generated kernels).
#pragma once

namespace afir {
namespace kernels {

// First statement of a kernel that may be launched with programmatic stream serialisation: it lets the next
// kernel of the stream be scheduled as soon as every CTA of this one has got this far, and then waits until
// everything before this kernel in the stream has completed and its writes are visible.  Nothing of global
// memory is touched before the wait, so the stream's order is the same as without the attribute; what is gained
// is that a kernel's launch and CTA start-up overlap the previous kernel's tail.  Both instructions do nothing in
// a kernel launched the ordinary way.
__device__ __forceinline__ void gridDependencyPrologue() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

} // namespace kernels
} // namespace afir
