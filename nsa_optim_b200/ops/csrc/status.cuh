// Error reporting without traps.  A kernel that gives up on a wait, or that finds an
// argument it cannot handle, writes one record into a KernelStatus block that lives in
// mapped pinned host memory and returns normally; the host checks the block after the
// next synchronisation and raises a Python exception.  The CUDA context stays usable.
#pragma once
#include <stdint.h>

struct KernelStatus {
  int code;    // 0 = ok; otherwise one of the STATUS_* values below (first failure wins)
  int block;   // blockIdx.x of the reporting CTA
  int info;    // kernel-specific detail (stage, parity, peer rank, ...)
  int count;   // number of reports since the last reset
};

enum : int {
  STATUS_OK = 0,
  STATUS_TIMEOUT_SMEM_FULL = 101,    // consumer never saw a TMA stage arrive
  STATUS_TIMEOUT_SMEM_EMPTY = 102,   // producer never got a stage back
  STATUS_TIMEOUT_TMEM_FULL = 103,    // epilogue never saw the accumulator complete
  STATUS_TIMEOUT_TMEM_EMPTY = 104,   // MMA warp never got an accumulator back
  STATUS_TIMEOUT_PEER_FLAG = 201,    // a flag written by another GPU never reached its value
  STATUS_TIMEOUT_LOCAL_FLAG = 202,   // a flag written by another CTA of this GPU never did
  STATUS_BAD_ARGUMENT = 301,
  STATUS_BAD_INDEX = 302,            // debug builds: an index read from a tensor was outside its range
};

#ifdef __CUDACC__
__device__ __forceinline__ void status_report(KernelStatus* st, int code, int block, int info) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->block = block;
    st->info = info;
  }
  atomicAdd(&st->count, 1);
  __threadfence_system();
}

// Debug builds (-DNSA_DEBUG_BOUNDS, `python -m nsa_optim_b200.ops.build --debug`): indices that
// kernels read from tensors (token ids, labels, selected-block numbers) are checked against their
// range where they are used.  A bad one is recorded (STATUS_BAD_INDEX, info = the index) and the
// kernel goes on with the clamped or skipped value it uses in release builds, so nothing faults;
// release builds compile the check away and clamp or skip silently.
#ifdef NSA_DEBUG_BOUNDS
#define NSA_CHECK_INDEX(ok, st, info) do { if (!(ok)) status_report((st), STATUS_BAD_INDEX, blockIdx.x, static_cast<int>(info)); } while (0)
#else
#define NSA_CHECK_INDEX(ok, st, info) do { } while (0)
#endif
#endif
