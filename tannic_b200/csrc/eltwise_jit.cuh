// Run-time instantiation of the fused element-wise row kernel for a caller's node list.
#pragma once

#include "common.cuh"

namespace tnb {

// A compiled instance of prog::ew_program_rows<T, P, UNROLL, ANY_SCALAR> whose P is the caller's
// program: straight-line code with every value in a register, like the programs compiled ahead
// of time, instead of the in-kernel interpreter.
struct JitKernel {
    void* function = nullptr;  // CUfunction
    int ctas_per_sm = 1;       // resident CTAs of 256 threads, from the occupancy calculator
};

// `elements`: size of the result (small results are not worth a compilation unless asked for).
// Returns the kernel for (dtype, node list, inputs, unroll, scalar-operand handling) on the current
// device, compiling it on first use (about a second; kept for the life of the process), or nullptr
// when run-time compilation is switched off, unavailable (no libnvrtc, no CUDA headers) or failed:
// the caller then runs the interpreter. Never returns a failure status for those reasons.
const JitKernel* jit_program_rows(int dtype, const tn_eltwise_node_t* nodes, int n_nodes, int n_inputs, int unroll, bool any_scalar, int64_t elements);

// Launches it with `args` pointing at the prog::ProgArgs of the call.
tn_status jit_launch(const JitKernel* kernel, unsigned grid_x, unsigned grid_y, void* args, cudaStream_t stream);

}  // namespace tnb
