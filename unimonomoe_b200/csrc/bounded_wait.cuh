// Global scratch ("workspace") layout, the status word, and every blocking wait of the
// kernel. All waits are bounded: when a wait exceeds the time limit it records
// (code, site, block) in the workspace status word, raises the grid-wide abort flag
// that every other wait polls, and returns false; the kernel then skips the remaining
// phases and returns normally, so the context stays usable and the host reads the
// status. The reference's waits are unbounded spins
// (kernel/moe_monokernel/src/moe_grid_barrier.h:101-199,
// kernel/qwen_tp/src/prefill_mono_final_nb.cu:244-247, :1468, :1500).
#pragma once
#include <cstddef>
#include <cstdint>
#include "ptx_sm100.cuh"

namespace mono {

constexpr int kGrid = 148;          // persistent CTAs, one per B200 SM
constexpr int kNumExperts = 256;    // experts the router scores
constexpr int kTpMaxChunks = 16;    // chunk cap of the fused tensor-parallel epilogue
constexpr int kBarrierSites = 8;

enum StatusCode : uint32_t {
  kStatusOk = 0,
  kErrGridBarrier = 1,   // a CTA did not reach a grid barrier in time
  kErrMbarrier = 2,      // a shared-memory pipeline barrier did not complete in time
  kErrChunkReady = 3,    // tensor-parallel: compute blocks did not finish a chunk in time
  kErrRankBarrier = 4,   // tensor-parallel: a peer rank did not arrive in time
  kErrDoneFlag = 5,      // tensor-parallel: final rank barrier not observed in time
  kErrBounds = 6,        // an index computed on the device fell outside its buffer
};

// Everything is a 4-byte word except the 8-byte time stamps at the (8-byte aligned) end. The words a launch
// needs at zero come first (kWorkspaceZeroBytes of them): the launcher clears only those; everything behind
// them is written in full by the kernel before it is read.
struct Workspace {
  uint32_t barrier[kBarrierSites];          // arrival counters, one per barrier site, used once per launch
  uint32_t status;                          // 0 = ok, else (code << 24) | (site << 16) | block
  uint32_t abort_flag;                      // raised together with status
  uint32_t status_aux[2];                   // free-form detail for the first error
  uint32_t tp_ready[kTpMaxChunks];          // compute blocks that finished chunk c
  uint32_t tp_open[kTpMaxChunks];           // 1 once every rank has finished chunk c (set behind the rank barrier)
  uint32_t tp_piece[kTpMaxChunks];          // next piece of this rank's share of chunk c to reduce
  uint32_t tp_pieces_done;                  // pieces reduced and made visible
  uint32_t tp_done_flag;                    // set once the final rank barrier is past
  uint32_t tp_seq_pub;                      // this launch's sequence number
  uint32_t reserved2;
  // ---- end of the part the launcher zeroes
  int32_t total_tiles;                      // tiles of 128 sorted rows in this launch
  int32_t reserved0[3];
  int32_t expert_counts[kNumExperts];       // rows routed to each local expert
  int32_t expert_offsets[kNumExperts + 1];  // exclusive prefix sum of expert_counts
  int32_t reserved1[3];
  int32_t cta_hist[kGrid][kNumExperts];     // per-CTA histograms (basis of the stable scatter)
  uint64_t phase_ns[8];                     // %globaltimer at phase boundaries, written by block 0
  uint64_t prof[kGrid][64];                 // per-CTA stall counters (cycles), filled only by MONO_PROFILE builds
};
constexpr size_t kWorkspaceZeroBytes = offsetof(Workspace, total_tiles);

struct WaitCtx {
  Workspace* ws;
  uint64_t timeout_ns;
};

__device__ __forceinline__ void report_error(Workspace* ws, uint32_t code, uint32_t site, uint32_t aux0 = 0,
                                             uint32_t aux1 = 0) {
  const uint32_t word = (code << 24) | ((site & 0xFFu) << 16) | (blockIdx.x & 0xFFFFu);
  if (atomicCAS(&ws->status, 0u, word) == 0u) {
    ws->status_aux[0] = aux0;
    ws->status_aux[1] = aux1;
  }
  __threadfence();
  atomicExch(&ws->abort_flag, 1u);
}

__device__ __forceinline__ bool aborted(const Workspace* ws) { return ld_relaxed_gpu(&ws->abort_flag) != 0u; }

// Wait for phase `parity` of a shared-memory barrier. False on abort or time-out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& c, uint32_t site) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 31u) == 0u) {
      if (aborted(c.ws)) return false;
      if (globaltimer_ns() - t0 > c.timeout_ns) {
        report_error(c.ws, kErrMbarrier, site, parity, threadIdx.x);
        return false;
      }
    }
  }
  return true;
}

// The same wait made by all 32 lanes of a converged warp with a warp-uniform result, so that the code after it
// stays convergent (the MMA warp: its tcgen05 instructions are issued by an elected lane out of uniform control
// flow, which lets the compiler keep descriptors and addresses in uniform registers).
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, const WaitCtx& c, uint32_t site) {
  if (__all_sync(0xFFFFFFFFu, mbar_try_wait(bar, parity))) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t polls = 0;
  while (!__all_sync(0xFFFFFFFFu, mbar_try_wait(bar, parity))) {
    if ((++polls & 31u) == 0u) {
      bool bad = false;
      if ((threadIdx.x & 31u) == 0u) {
        if (aborted(c.ws)) bad = true;
        else if (globaltimer_ns() - t0 > c.timeout_ns) {
          report_error(c.ws, kErrMbarrier, site, parity, threadIdx.x);
          bad = true;
        }
      }
      if (__any_sync(0xFFFFFFFFu, bad)) return false;
    }
  }
  return true;
}

// Spin until *p >= target (device scope). False on abort or time-out.
__device__ __forceinline__ bool wait_counter_ge(const uint32_t* p, uint32_t target, const WaitCtx& c,
                                                uint32_t code, uint32_t site) {
  if (ld_acquire_gpu(p) >= target) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t polls = 0;
  for (;;) {
    const uint32_t v = ld_acquire_gpu(p);
    if (v >= target) return true;
    if ((++polls & 7u) == 0u) {
      if (aborted(c.ws)) return false;
      if (globaltimer_ns() - t0 > c.timeout_ns) {
        report_error(c.ws, code, site, v, target);
        return false;
      }
    }
    __nanosleep(40);
  }
}

// Grid-wide barrier over kGrid co-resident CTAs. Each site has its own counter that
// the launcher zeroes, and is used once per launch. Returns false (in every thread of
// the CTA) when the launch is aborting.
__device__ __forceinline__ bool grid_sync(const WaitCtx& c, int site, uint32_t* s_flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(&c.ws->barrier[site], 1u);
    const bool ok = wait_counter_ge(&c.ws->barrier[site], static_cast<uint32_t>(kGrid), c, kErrGridBarrier,
                                    static_cast<uint32_t>(site));
    __threadfence();
    *s_flag = ok ? 1u : 0u;
  }
  __syncthreads();
  return *s_flag != 0u;
}

}  // namespace mono
