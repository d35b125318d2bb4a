// Stand-in for <hip/hip_runtime.h> that lets the reference's kernel templates compile as host C++.
// TEST INFRASTRUCTURE ONLY (see oracle/build_ref.py): the kernels under
// vte/compiler/templates/rdna/ are compiled from where they lie in the reference checkout and run
// on CPU threads, one std::thread per GPU thread of a block, blocks one after another.
// Only what those templates use is here: the launch-geometry variables, __syncthreads (a barrier
// over the block's threads), __expf, min.  `extern __shared__` / `__shared__` are rewritten to
// `extern` / `static` by the build recipe (one block runs at a time, so a process-wide array is
// the block's shared memory).
#pragma once
#include <cmath>
#include <cstddef>
#include <algorithm>

struct dim3 {
    unsigned x, y, z;
};
extern thread_local dim3 threadIdx;
extern dim3 blockIdx, blockDim, gridDim;
extern float smem[];                       // the dynamic shared memory of the block in flight

void vte_ref_block_barrier();
inline void __syncthreads() { vte_ref_block_barrier(); }
inline float __expf(float x) { return std::exp(x); }
using std::min;
using std::max;

#define __global__
#define __device__
#define __forceinline__ inline
#define __restrict__ __restrict
