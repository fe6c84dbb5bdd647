// Programmatic dependent launch (griddepcontrol) for the kernels of a decode step.
#pragma once

namespace ti {

// A kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization may start while the kernel
// before it in the stream is still running, as soon as every CTA of that kernel has executed
// grid_dep_launch() (or exited).  It must execute grid_dep_wait() before it reads anything the earlier
// kernel wrote or writes anything the earlier kernel reads: the wait returns when the earlier kernel has
// completed and its memory operations are visible.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace ti
