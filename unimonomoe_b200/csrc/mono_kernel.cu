// Single-launch FP8 MoE prefill layer for B200 (sm_100a): one persistent kernel, 148
// CTAs (one per SM), phases separated by bounded software grid barriers.
//
//   phase R   (only through the _gemv entry) router logits = x * W_r^T on the tensor cores:
//             bf16 x bf16 -> fp32, every CTA for the tokens it routes itself
//   phase 0   router top-k from fp32 logits (softmax, sigmoid+bias, or group-limited
//             sigmoid+bias), per-warp expert histograms; bf16 -> e4m3 activation
//             quantisation with one fp32 scale per (token, 128 columns)
//   phase 1   prefix sum over experts, tile schedule, STABLE counting-sort scatter
//   phase 2   per tile of <=128 sorted rows of one expert, warp-specialised:
//               TMA warp      block-FP8 weight tiles -> shared memory (SWIZZLE_128B)
//               gather warps  the tile's e4m3 activation rows -> shared memory (cp.async)
//               MMA thread    tcgen05.mma kind::f8f6f4, M=128 N=256 K=32, one 128-deep
//                             K slab at a time into one of two 256-column TMEM buffers
//               8 epilogue warps  tcgen05.ld each slab, fold w_scale*a_scale into fp32
//                             register accumulators, SiLU(gate)*up, requantise to e4m3
//                             per (row,128) into shared memory, which the MMA thread
//                             then uses as the A operand of the down projection; the
//                             down result times the routing weight goes out as bf16
//   phase 3   per token sum of its top-k partial rows -> bf16 [T,H]; under tensor or expert
//             parallelism a chunked one-shot all-reduce of the ranks' outputs runs in the same
//             launch: the last `ncomm` CTAs open finished chunks (rank barrier) and reduce them
//             through the NVLS multicast alias (two ranks: by direct peer loads) while the others
//             still sum, and every summing CTA joins the transfer when its sums are done.
//
// An intermediate wider than 512 columns is processed in chunks of 512 (one partial row per chunk);
// -DMONO_PAIR=1 schedules pairs of tiles on clusters of two CTAs (tcgen05 cta_group::2).
//
// What it replaces in the reference (same semantics, different machine):
//   kernel/qwen_tp/src/prefill_mono_final_nb.cu:932-1506 (device kernel),
//   :1513-1791 (host launcher and accessors), kernel/qwen_ep/src/...:1185-1207,
//   :1373-1379, :1459-1481 (expert-parallel ownership), kernel/deepseek_tp/src/...
//   (geometry and router mode). Geometry is fixed at compile time through the MONO_*
//   macros and read back through the prefill_wgmma_* accessors.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "bounded_wait.cuh"
#include "pair_sm100.cuh"
#include "ptx_sm100.cuh"
#include "route_math.cuh"

#ifndef MONO_K_DIM
#define MONO_K_DIM 2048
#endif
#ifndef MONO_H_DIM
#define MONO_H_DIM 2048
#endif
#ifndef MONO_N_HALF
#define MONO_N_HALF 512
#endif
#ifndef MONO_E_LOCAL
#define MONO_E_LOCAL 256
#endif
#ifndef MONO_ROUTER_MODE
#define MONO_ROUTER_MODE 0
#endif

// Development only: MONO_ABLATE is a bit mask that removes a piece of the epilogue's work (the
// results are then wrong) so that its share of the run time can be measured by difference.
//   1: no TMEM read-out / promotion   2: no SiLU / requantisation arithmetic   4: no partial-row stores
//   8: no activation gather copies    16: no weight TMA loads
//   256: no lane exchange before the partial-row stores (same bytes, wrong columns)
//   128: every slab step issues its four MMAs twice (1024 tensor-core cycles per step: is a step bound by latency or by issue?)
//   64: no operand hand-shake at all (producers idle; the MMA warp waits only for accumulator buffers)
//   32: the intermediate's passes alias one 16 KB slot, which leaves room for four-deep operand rings
#ifndef MONO_ABLATE
#define MONO_ABLATE 0
#endif
#ifndef MONO_MMA_WARP
#define MONO_MMA_WARP 1
#endif

// Development only: MONO_TRACE (with MONO_PROFILE) makes CTA 0 write clock64 time stamps of its MMA thread
// (5 per slab step: top, operands B, operands A, accumulator free, issued) and of epilogue thread 0 (4 per step:
// before the wait, after it, buffer released, folded) over the stall-counter area, for a timeline of the hand-shake.
#if defined(MONO_TRACE) && defined(MONO_PROFILE)
#define TRACE_M(k) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && tr_m < 4000) reinterpret_cast<unsigned long long*>(p.ws->prof)[tr_m++] = clock64(); } while (0)
#define TRACE_E(k) do { if (blockIdx.x == 0 && et == 0 && tr_e < 8000) reinterpret_cast<unsigned long long*>(p.ws->prof)[tr_e++] = clock64(); } while (0)
#else
#define TRACE_M(k)
#define TRACE_E(k)
#endif

#ifdef MONO_PROFILE
#define PROF_DECL(n) long long n = 0
#define PROF_T0() const long long prof_t0_ = clock64()
#define PROF_ADD(n) n += clock64() - prof_t0_
#ifdef MONO_TRACE
#define PROF_STORE(slot, n)
#else
#define PROF_STORE(slot, n) p.ws->prof[blockIdx.x][slot] = static_cast<uint64_t>(n)
#endif
#define PROF_HIST(row, bin, who) do { if (who) S.whist[row][bin] += static_cast<unsigned long long>(clock64() - prof_t0_); } while (0)
#else
#define PROF_DECL(n)
#define PROF_T0()
#define PROF_ADD(n)
#define PROF_STORE(slot, n)
#define PROF_HIST(row, bin, who)
#endif

namespace mono {
namespace {

// ------------------------------------------------------------------ geometry
constexpr int E = kNumExperts;
constexpr int E_LOCAL = MONO_E_LOCAL;
constexpr bool EP_BUILD = (E_LOCAL != E);
constexpr int TOP_K = 8;
constexpr int K_DIM = MONO_K_DIM;
constexpr int H_DIM = MONO_H_DIM;
constexpr int N_HALF = MONO_N_HALF;
constexpr int N_UP = 2 * N_HALF;
constexpr int ROUTER_MODE = MONO_ROUTER_MODE;
constexpr int N_GROUP = 8;
constexpr int TOPK_GROUP = 4;
constexpr int NK = K_DIM / 128;    // K slabs of the up projection
// An intermediate wider than 512 columns does not fit in shared memory as one e4m3 tile, so a tile is
// then processed in NCH chunks of 512 intermediate columns. Each (tile, chunk) is an independent unit of
// work: up projection of the chunk's gate/up columns, SiLU, requantisation, and the down projection over
// the chunk's K range, which yields its own bf16 partial row; the slot sum adds top_k * NCH rows per token.
constexpr int NPT = N_HALF / 128;  // 128-column blocks of the whole intermediate
constexpr int CHUNK_COLS = N_HALF > 512 ? 512 : N_HALF;
constexpr int NCH = N_HALF / CHUNK_COLS;
constexpr int NP = CHUNK_COLS / 128;  // 128-column passes of the up projection = K slabs of the down projection, per chunk
static_assert(N_HALF % CHUNK_COLS == 0, "the intermediate splits into whole chunks");
static_assert(CHUNK_COLS / 128 <= 4, "one intermediate-ready barrier per pass: at most four passes");
constexpr int NHB = H_DIM / 256;   // 256-column passes of the down projection
constexpr int TILE_M = 128;

static_assert(E == 256, "routing keeps 8 logits per lane: exactly 256 experts");
static_assert(E_LOCAL > 0 && E_LOCAL <= E, "local experts are a subset");
static_assert(K_DIM % 128 == 0 && N_HALF % 128 == 0 && H_DIM % 256 == 0, "geometry must tile by 128/256");
static_assert(ROUTER_MODE >= 0 && ROUTER_MODE <= 2, "unknown router mode");
static_assert(NK % 2 == 0, "activation quantisation pairs two 128-column groups per warp");
static_assert(ROUTER_MODE != 2 || N_GROUP * 32 == E, "grouped routing assumes 32 experts per group");

// ------------------------------------------------------------------ launch shape
// Warps 0-3 are the producer warpgroup (weight TMA, MMA issue, two gather warps); the epilogue is
// EPI_WGS warpgroups of 128 threads. Thread i of an epilogue warpgroup owns row i of the tile
// (TMEM lane i); warpgroup h owns columns [h*WC, (h+1)*WC) of every accumulator buffer: HCB gate
// columns followed by the HCB matching up columns in the up projection, WC output columns in
// the down projection.
#ifndef MONO_EPI_WGS
#define MONO_EPI_WGS 2
#endif
#ifndef MONO_NSPLIT
#define MONO_NSPLIT 1
#endif
// MONO_PAIR=1: tiles are scheduled as pairs of 128-row tiles of one expert on a cluster of two CTAs
// (tcgen05 cta_group::2, M = 256). Each CTA gathers its own 128 activation rows and loads HALF of every
// weight stage; one thread of the cluster's rank-0 CTA issues the MMAs for both. Halves the weight
// bytes every SM pulls from L2 and makes room for deeper operand rings.
#ifndef MONO_PAIR
#define MONO_PAIR 0
#endif
constexpr bool PAIR = MONO_PAIR != 0;
constexpr int EPI_WGS = MONO_EPI_WGS;
static_assert(EPI_WGS == 2 || EPI_WGS == 4, "two or four epilogue warpgroups");
static_assert(!PAIR || (EPI_WGS == 2 && MONO_NSPLIT == 1), "the pair schedule is written for two epilogue warpgroups, N = 256");
// A 128-deep K slab of the 256 weight rows of a stage is issued as NSPLIT independent MMAs of
// N = BC columns, each into its own TMEM buffer, so the epilogue's read-out of one buffer is a
// single short dependency chain and the MMA thread can run NBUF-1 buffers ahead of it.
constexpr int NSPLIT = MONO_NSPLIT;
constexpr int BC = 256 / NSPLIT;         // columns of one accumulator buffer = N of one MMA
constexpr int NBUF = 2 * NSPLIT;         // accumulator buffers in tensor memory (512 columns in all)
constexpr int WC = BC / EPI_WGS;         // columns of one buffer owned by one epilogue warpgroup
constexpr int HCB = WC / 2;              // gate (= up) columns per warpgroup per buffer
constexpr int TCOLS = NSPLIT * WC;       // accumulator columns (fp32 registers) per epilogue thread
constexpr int PASS_STRIDE = 128 / NSPLIT;  // intermediate columns covered by one buffer in the up projection
constexpr int LDW = (WC <= 64) ? WC : HCB;  // TMEM columns per tcgen05.ld
constexpr int NLD = WC / LDW;
static_assert(HCB == 32 || HCB == 64, "unsupported split of the accumulator between warpgroups");
static_assert(LDW == 32 || LDW == 64, "TMEM loads are 32 or 64 columns wide");
constexpr int N_EPI = EPI_WGS * 128;
constexpr int BLOCK = 128 + N_EPI;
constexpr int NWARPS = BLOCK / 32;
constexpr int WARP_TMA = 0, WARP_MMA = 1, WARP_GATHER0 = 2;  // warps 2,3 gather; warps 4.. epilogue
constexpr int N_GATHER = 64;
constexpr int MAX_MY_TILES = 32 * NCH;
constexpr int MAX_TILES = MAX_MY_TILES * kGrid;

// ------------------------------------------------------------------ shared memory plan
constexpr int A_STAGE_BYTES = TILE_M * 128;  // 128 rows x 128 B
constexpr int B_ROWS = PAIR ? 128 : 256;     // weight rows of a stage kept by one CTA
constexpr int B_STAGE_BYTES = B_ROWS * 128;  // x 128 B
constexpr int STAGE_CAP = PAIR ? 6 : 4;
constexpr int INTER_SLOTS = (MONO_ABLATE & 32) ? 1 : NP;  // ablation 32: all passes share one slot (deeper rings, wrong results)
constexpr int INTER_BYTES = INTER_SLOTS * A_STAGE_BYTES;
constexpr int SMEM_CAP = 227 * 1024;
constexpr int SMEM_STATIC_RESERVE = 6 * 1024;
// per-tile scale staging: activation scales [NK][128], and (double buffered) the expert's
// up-projection scales [2*NP*NK] and down-projection scales [(H/128)*NP]
constexpr int WSU_N = 2 * NP * NK;
constexpr int WSD_N = (H_DIM / 128) * NP;
constexpr int SCALE_BYTES = ((NK * TILE_M + 2 * WSU_N + 2 * WSD_N) * 4 + 1023) / 1024 * 1024;
constexpr int AS_PIECES = NK / 8;  // 16-byte pieces of activation scales each epilogue thread stages per tile
static_assert(NK % 8 == 0, "each epilogue thread stages NK/2 activation scales in 16-byte pieces");
static_assert(NHB >= AS_PIECES + 2, "the next tile's scales are staged during the down projection");
constexpr int SMEM_AVAIL = SMEM_CAP - SMEM_STATIC_RESERVE - 1024 - INTER_BYTES - SCALE_BYTES;
constexpr int SB_RAW = SMEM_AVAIL / (A_STAGE_BYTES + B_STAGE_BYTES);
constexpr int SB = SB_RAW > STAGE_CAP ? STAGE_CAP : SB_RAW;
constexpr int SA_RAW = (SMEM_AVAIL - SB * B_STAGE_BYTES) / A_STAGE_BYTES;
constexpr int SA = SA_RAW > STAGE_CAP ? STAGE_CAP : SA_RAW;
static_assert(SB >= 2 && SA >= 2, "intermediate too wide for shared memory: shard N_HALF further");
constexpr int DYN_SMEM = 1024 + INTER_BYTES + SA * A_STAGE_BYTES + SB * B_STAGE_BYTES + SCALE_BYTES;
static_assert(NWARPS * E * 4 <= SA * A_STAGE_BYTES, "phase-0 histograms live in the activation ring");

// Register budget (setmaxnreg). The kernel launches with REGS_LAUNCH registers per thread; the
// producer warpgroup gives registers back and the epilogue warpgroups take them. The
// hardware hands out only what this CTA released, and setmaxnreg.inc waits (without a bound)
// until it is available, so the three counts MUST satisfy the inequality below.
constexpr int REGS_LAUNCH = (65536 / BLOCK) / 8 * 8;            // 168 at 384 threads, 96 at 640
#ifndef MONO_REGS_PRODUCER
#define MONO_REGS_PRODUCER 56
#endif
constexpr int REGS_PRODUCER = (EPI_WGS == 2) ? MONO_REGS_PRODUCER : 40;
constexpr int REGS_EPILOGUE = ((BLOCK * REGS_LAUNCH - 128 * REGS_PRODUCER) / N_EPI) / 8 * 8;  // 224 / 104
static_assert(128 * REGS_PRODUCER + N_EPI * REGS_EPILOGUE <= BLOCK * REGS_LAUNCH,
              "setmaxnreg.inc would wait forever: the epilogue asks for more registers than the producers release");
static_assert(REGS_LAUNCH * BLOCK <= 65536, "launch register count exceeds the register file");

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t IDESC = umma_idesc_e4m3_f32(PAIR ? 256 : 128, BC);
// router GEMV: one [128 tokens x 256 experts] accumulator, K slabs of 64 bf16 (128 bytes)
constexpr uint32_t IDESC_ROUTER = umma_idesc_bf16_f32(128, E);
constexpr int RK = K_DIM / 64;
constexpr int RS = (SA < SB) ? SA : SB;

// wait sites reported in the status word
enum Site : uint32_t {
  kSiteEmptyB = 1, kSiteFullB, kSiteFullA, kSiteEmptyA, kSiteTmemEmpty, kSiteTmemFull, kSiteInterReady,
  kSiteRouterEmpty, kSiteRouterFull, kSiteRouterAccEmpty, kSiteRouterAccFull,
};

struct Params {
  const float* logits;
  int num_tokens;
  Workspace* ws;
  int32_t* topk_ids;
  float* topk_weights;
  int32_t* sorted_ids;
  const __nv_bfloat16* act_bf16;
  uint8_t* act_fp8;
  float* act_scales;
  const float* up_w_scales;
  const float* down_w_scales;
  __nv_bfloat16* partial;   // [T*8, H] bf16 partial rows (the caller's output_accum buffer)
  __nv_bfloat16* out;       // [T, H]
  const float* router_bias;
  const int32_t* expert_map;
  // tensor-parallel epilogue
  __nv_bfloat16* tp_mc;
  uint32_t** tp_pads;
  int tp_rank, tp_world, tp_nchunk, tp_ncomm;
  uint32_t tp_seq;
  uint32_t* tp_seqctr;
  __nv_bfloat16** tp_peers;   // every rank's address of the output window (device array), or null
  const __nv_bfloat16* residual;
  float out_scale;
  uint64_t timeout_ns;
  // optional debug dump (null in production): raw gate|up accumulators, e4m3 intermediate, its scales
  float* dbg_acc;
  uint8_t* dbg_inter;
  float* dbg_inter_scale;
  // shared expert computed in the same launch (sh_on == 0: none). Its tiles are the token tiles j with
  // j % sh_parts == sh_part; its partial rows follow the routed ones in `partial`.
  const float* sh_up_scales;
  const float* sh_down_scales;
  const __nv_bfloat16* sh_gate;   // [K] gate vector (sigmoid(x . g) scales the row), or null: weight 1
  float* sh_gate_w;               // [T] fp32, written by phase 0 when sh_gate is given
  int sh_on, sh_part, sh_parts;
  // router GEMV (null: the caller supplied the logits)
  float* logits_out;        // [T, E] fp32, written by phase R and read back by phase 0
  alignas(64) CUtensorMap tm_up;
  alignas(64) CUtensorMap tm_down;
  alignas(64) CUtensorMap tm_x;    // bf16 activations [T, K]
  alignas(64) CUtensorMap tm_rw;   // bf16 router weight [E, K]
  alignas(64) CUtensorMap tm_sh_up;    // shared expert [2 * N_HALF, K]
  alignas(64) CUtensorMap tm_sh_down;  // shared expert [H, N_HALF]
};

// e == SHARED_E marks a tile of the shared expert: its rows are the tokens row0 .. row0 + rows - 1 themselves
// (no sort indirection), its weights the shared expert's.
struct TileInfo {
  int e, row0, rows, chunk;
};
constexpr int SHARED_E = E_LOCAL;

// ------------------------------------------------------------------ small helpers
__device__ __forceinline__ uint32_t float_key(float f) {
  // Monotone map float -> uint32 for finite values; 0 is reserved for "not selectable".
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long k) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xFFFFFFFFu, k, off);
    k = o > k ? o : k;
  }
  return k;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
  return v;
}
// Byte offset of 16-byte chunk c of row r inside a [rows x 128 B] tile in the 128-byte
// swizzle: eight-row groups of 1024 B, chunk position XORed with the row's low 3 bits.
__device__ __forceinline__ uint32_t sw128(int r, int c) {
  return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// ------------------------------------------------------------------ phase 0: routing
// One warp per token. Lane l holds experts l, l+32, ..., l+224; register slot j therefore
// spans experts [32j, 32j+32), which is one DeepSeek expert group.
// Semantics follow kernel/qwen_tp/src/prefill_mono_final_nb.cu:1025-1185: selection in
// descending score order, ties to the lower expert id, weights renormalised by their sum
// (clamped at 1e-30); modes 1/2 select on sigmoid+bias and weight by the unbiased sigmoid.
// A slot for which no selectable expert remains gets id -1 and weight 0.
// NT tokens are routed side by side (every step loops over them) so that the shuffle / redux / division
// latencies of one token are filled with the other's instructions; the arithmetic per token is unchanged.
template <int NT>
__device__ __forceinline__ void route_tokens(const float (&logit)[NT][8], const float* __restrict__ bias, int lane,
                                             int (&my_id)[NT], float (&my_w)[NT]) {
  float sel[NT][8], unb[NT][8];
  float m[NT], s[NT];
#pragma unroll
  for (int a = 0; a < NT; ++a) {
    m[a] = 0.f;
    s[a] = 1.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) sel[a][j] = logit[a][j];
  }
  if constexpr (ROUTER_MODE == 0) {
#pragma unroll
    for (int a = 0; a < NT; ++a) {
      m[a] = sel[a][0];
#pragma unroll
      for (int j = 1; j < 8; ++j) m[a] = fmaxf(m[a], sel[a][j]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int a = 0; a < NT; ++a) m[a] = fmaxf(m[a], __shfl_xor_sync(0xFFFFFFFFu, m[a], off));
    }
    float part[NT];
#pragma unroll
    for (int a = 0; a < NT; ++a) {
      part[a] = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) part[a] += det_expf(sel[a][j] - m[a]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int a = 0; a < NT; ++a) part[a] += __shfl_xor_sync(0xFFFFFFFFu, part[a], off);
    }
#pragma unroll
    for (int a = 0; a < NT; ++a) {
      s[a] = part[a];
#pragma unroll
      for (int j = 0; j < 8; ++j) unb[a][j] = sel[a][j];
    }
  } else {
#pragma unroll
    for (int a = 0; a < NT; ++a) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = det_sigmoidf(sel[a][j]);
        unb[a][j] = sg;
        sel[a][j] = (bias != nullptr) ? __fadd_rn(sg, bias[lane + 32 * j]) : sg;
      }
    }
    if constexpr (ROUTER_MODE == 2) {
#pragma unroll
      for (int a = 0; a < NT; ++a) {
        float gs[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // top-1 (with its lane, ties to the lower lane) and top-2 of the group
          const bool ok = sel[a][j] > -FLT_MAX;
          unsigned long long k1 = ok ? ((static_cast<unsigned long long>(float_key(sel[a][j])) << 32) |
                                        static_cast<unsigned long long>(31 - lane))
                                     : 0ull;
          k1 = warp_max_u64(k1);
          const int l1 = 31 - static_cast<int>(k1 & 0xFFFFFFFFull);
          const float b1 = __shfl_sync(0xFFFFFFFFu, sel[a][j], l1 & 31);
          float b2 = (lane == l1 || !ok) ? -FLT_MAX : sel[a][j];
          b2 = warp_max_f(b2);
          gs[j] = (k1 == 0ull) ? -FLT_MAX : __fadd_rn(b1, b2);
        }
        uint32_t keep = 0u;
#pragma unroll
        for (int r = 0; r < TOPK_GROUP; ++r) {
          float gb = -FLT_MAX;
          int gi = -1;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (!((keep >> j) & 1u) && gs[j] > gb) { gb = gs[j]; gi = j; }
          if (gi >= 0) keep |= 1u << gi;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (!((keep >> j) & 1u)) sel[a][j] = -FLT_MAX;
      }
    }
  }

  // One 32-bit orderable key per candidate, built once; 0 = not selectable / taken. A round takes the
  // largest key of the warp (redux.sync.max) and, among the candidates that carry it, the lowest expert
  // id (redux.sync.min): descending score, ties to the lower id.
  uint32_t key[NT][8];
  float wsum[NT];
#pragma unroll
  for (int a = 0; a < NT; ++a) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = sel[a][j] + 0.0f;  // folds -0 into +0 so that the integer key orders exactly like operator>
      key[a][j] = (v > -FLT_MAX) ? float_key(v) : 0u;
    }
    wsum[a] = 0.f;
    my_id[a] = -1;
    my_w[a] = 0.f;
  }
#pragma unroll 1
  for (int k = 0; k < TOP_K; ++k) {
    uint32_t best[NT];
    int bidx[NT];
    float mine[NT];
#pragma unroll
    for (int a = 0; a < NT; ++a) {
      const uint32_t m01 = max(key[a][0], key[a][1]), m23 = max(key[a][2], key[a][3]),
                     m45 = max(key[a][4], key[a][5]), m67 = max(key[a][6], key[a][7]);
      best[a] = __reduce_max_sync(0xFFFFFFFFu, max(max(m01, m23), max(m45, m67)));
    }
#pragma unroll
    for (int a = 0; a < NT; ++a) {
      uint32_t cand = 0xFFFFFFFFu;
#pragma unroll
      for (int j = 7; j >= 0; --j)
        if (key[a][j] == best[a] && best[a] != 0u) cand = static_cast<uint32_t>(lane + 32 * j);
      bidx[a] = static_cast<int>(__reduce_min_sync(0xFFFFFFFFu, cand));  // -1 when nothing is selectable
    }
#pragma unroll
    for (int a = 0; a < NT; ++a) {
      const int owner = bidx[a] & 31, slot = (bidx[a] >> 5) & 7;
      mine[a] = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j == slot && bidx[a] >= 0) {
          mine[a] = unb[a][j];
          if (lane == owner) key[a][j] = 0u;  // the owner retires the winner
        }
      }
      mine[a] = __shfl_sync(0xFFFFFFFFu, mine[a], owner);
      // lane k keeps the k-th winner and its unbiased score; the weights are formed after the loop, by the
      // eight lanes at once instead of one exponential and one division per round
      if (lane == k) { my_id[a] = bidx[a]; my_w[a] = mine[a]; }
    }
  }
#pragma unroll
  for (int a = 0; a < NT; ++a) {
    float wk = 0.f;
    if (lane < TOP_K && my_id[a] >= 0)
      wk = (ROUTER_MODE == 0) ? __fdiv_rn(det_expf(my_w[a] - m[a]), s[a]) : my_w[a];
    // the sum runs over the slots in ascending order, as a sequential accumulation would
    wsum[a] = 0.f;
#pragma unroll
    for (int k = 0; k < TOP_K; ++k) wsum[a] += __shfl_sync(0xFFFFFFFFu, wk, k);
    const float inv = __fdiv_rn(1.0f, fmaxf(wsum[a], 1e-30f));
    my_w[a] = __fmul_rn(wk, inv);
  }
}

// ------------------------------------------------------------------ phase 0.5: activation quantisation
// bf16 -> e4m3 with one fp32 scale per (token, 128 columns): amax, inv = 448/amax,
// q = e4m3_rn_satfinite(x * inv), scale = amax/448; amax < FLT_MIN is treated as 1
// (kernel/qwen_tp/src/prefill_mono_final_nb.cu:1225-1244). A half-warp owns one group.
// One token is quantised by one warp, in two steps so that the loads can be in flight while the
// warp does something else (routing): half-warp `half` owns the 128-column groups 2*u + half, lane `sub`
// of it the 16-byte piece `sub` of a group. A piece of work is QU groups per half-warp.
constexpr int QU = 8;
constexpr int Q_PIECES = (NK / 2 + QU - 1) / QU;
__device__ __forceinline__ void quant_token_load(const Params& p, int tok, int piece, int lane, uint4 (&raw)[QU]) {
  const int half = lane >> 4, sub = lane & 15;
#pragma unroll
  for (int u = 0; u < QU; ++u) {
    const int kb = 2 * (piece * QU + u) + half;
    raw[u] = make_uint4(0u, 0u, 0u, 0u);
    if (kb < NK)
      raw[u] = *reinterpret_cast<const uint4*>(p.act_bf16 + static_cast<size_t>(tok) * K_DIM + kb * 128 + sub * 8);
  }
}
// GATE: `gdot` also collects this lane's part of x . g for the shared expert's gate (a compile-time switch, so
// that launches without a gated shared expert run exactly the code they ran before there was one).
template <bool GATE>
__device__ __forceinline__ void quant_token_store(const Params& p, int tok, int piece, int lane, const uint4 (&raw)[QU],
                                                  const __nv_bfloat16* g, float& gdot) {
  const int half = lane >> 4, sub = lane & 15;
#pragma unroll
  for (int u = 0; u < QU; ++u) {
    const int kb = 2 * (piece * QU + u) + half;
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&raw[u]);
    float x[8];
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x[i] = __bfloat162float(b[i]);
      am = fmaxf(am, fabsf(x[i]));
    }
    if (GATE && kb < NK) {
      const uint4 gr = __ldg(reinterpret_cast<const uint4*>(g + kb * 128 + sub * 8));
      const __nv_bfloat16* gb = reinterpret_cast<const __nv_bfloat16*>(&gr);
#pragma unroll
      for (int i = 0; i < 8; ++i) gdot = __fmaf_rn(x[i], __bfloat162float(gb[i]), gdot);
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, off));
    if (am < FLT_MIN) am = 1.f;
    const float inv = __fdiv_rn(448.0f, am);
    if (kb < NK) {
      uint2 q;
      q.x = pack_e4m3x4(__fmul_rn(x[0], inv), __fmul_rn(x[1], inv), __fmul_rn(x[2], inv), __fmul_rn(x[3], inv));
      q.y = pack_e4m3x4(__fmul_rn(x[4], inv), __fmul_rn(x[5], inv), __fmul_rn(x[6], inv), __fmul_rn(x[7], inv));
      *reinterpret_cast<uint2*>(p.act_fp8 + static_cast<size_t>(tok) * K_DIM + kb * 128 + sub * 8) = q;
      if (sub == 0) p.act_scales[static_cast<size_t>(tok) * NK + kb] = __fdiv_rn(am, 448.0f);
    }
  }
}

// Position, in the expert's scale tensors, of entry i of the per-chunk staging arrays:
// up scales [2 * NPT, NK] -> staged [gate NP rows | up NP rows] x NK; down scales [H/128, NPT] -> staged [H/128, NP].
__device__ __forceinline__ size_t wsu_index(int e, int chunk, int i) {
  const int half = i / (NP * NK), rem = i % (NP * NK);
  return static_cast<size_t>(e) * (2 * NPT * NK) + static_cast<size_t>(half * NPT + chunk * NP) * NK + rem;
}
__device__ __forceinline__ size_t wsd_index(int e, int chunk, int i) {
  const int hb = i / NP, dk = i % NP;
  return static_cast<size_t>(e) * ((H_DIM / 128) * NPT) + static_cast<size_t>(hb) * NPT + chunk * NP + dk;
}

// ------------------------------------------------------------------ shared state
struct __align__(16) SharedState {
  uint64_t fullA[STAGE_CAP], emptyA[STAGE_CAP], fullB[STAGE_CAP], emptyB[STAGE_CAP];
  uint64_t tmem_full[NBUF], tmem_empty[NBUF];
  uint64_t inter_ready[4];  // one per 128-column pass of the intermediate (NP <= 4)
  uint64_t rfull[4], rempty[4], racc_full, racc_empty;  // phase R only
  uint32_t tmem_base;
  uint32_t flag;          // grid_sync result broadcast
  int n_my_tiles;
  int total_tiles;
  TileInfo tiles[MAX_MY_TILES];
  float rowmax[2][EPI_WGS][TILE_M];
  alignas(16) int gather_tok[2][8][TILE_M / 8];  // token of row gr + 8 i of the tile being gathered, [tile parity][gr][i]
#ifdef MONO_PROFILE
  // wait cycles by position of the slab step inside its pass: [0,16) up-projection slab ks, [16,20) down-projection slab dk;
  // one row for the epilogue's waits for a full accumulator, one for the MMA thread's waits for a free one
  unsigned long long whist[2][24];
#endif
};
static_assert(sizeof(SharedState) <= SMEM_STATIC_RESERVE, "static shared state exceeds its reserve");

// ------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(BLOCK, 1) moe_prefill_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t dyn_raw[];
  __shared__ SharedState S;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bid = blockIdx.x;
  const WaitCtx wc{p.ws, p.timeout_ns};
  Workspace* ws = p.ws;
  const int T = p.num_tokens;
  const int numel = T * TOP_K;

  // 1024-byte aligned base of the operand buffers
  const uint32_t dyn_u32 = (smem_u32(dyn_raw) + 1023u) & ~1023u;
  uint8_t* dyn = dyn_raw + (dyn_u32 - smem_u32(dyn_raw));
  uint8_t* inter = dyn;
  uint8_t* a_ring = dyn + INTER_BYTES;
  uint8_t* b_ring = a_ring + SA * A_STAGE_BYTES;
  float* as_sm = reinterpret_cast<float*>(b_ring + SB * B_STAGE_BYTES);  // [NK][128]
  float* wsu_sm = as_sm + NK * TILE_M;                                    // [2][WSU_N]
  float* wsd_sm = wsu_sm + 2 * WSU_N;                                     // [2][WSD_N]
  int* hist = reinterpret_cast<int*>(a_ring);  // [NWARPS][E], phases 0-1 only
  int* scan_cnt = reinterpret_cast<int*>(b_ring);  // phase 1 only: four arrays of E ints
  int* scan_tile = scan_cnt + E;
  int* ph1_tot = scan_tile + E;
  int* ph1_pre = ph1_tot + E;

  if (bid == 0 && tid == 0) ws->phase_ns[0] = globaltimer_ns();

  // launch sequence of the tensor-parallel epilogue: a device counter outside the
  // workspace (which is zeroed every launch) so that CUDA-graph replays advance it
  // (kernel/qwen_tp/src/prefill_mono_final_nb.cu:985-1016)
  const bool tp_on = (p.tp_mc != nullptr) && (p.tp_pads != nullptr) && (p.tp_ncomm > 0);
  if (tp_on && p.tp_seqctr != nullptr && bid == 0 && tid == 0) {
    const uint32_t sq = atomicAdd(p.tp_seqctr, 1u) + 1u;
    atomicExch(&ws->tp_seq_pub, sq);
  }

  // Every warp routes a contiguous range of tokens, so a CTA routes one contiguous range as well.
  const int gwarp = bid * NWARPS + warp;
  const int nwarps_grid = kGrid * NWARPS;
  const int tok_per_warp = (T + nwarps_grid - 1) / nwarps_grid;
  const int t_begin = min(T, gwarp * tok_per_warp);
  const int t_end = min(T, t_begin + tok_per_warp);

  // ================================================================ phase R (router GEMV)
  // logits[t, e] = sum_k x[t, k] * W_r[e, k] for the tokens THIS CTA routes in phase 0, so no grid
  // barrier separates the two. bf16 products are exact in fp32; the accumulation runs in the tensor
  // core's fp32 accumulator over K slabs of 64 in ascending order (its order inside one instruction is
  // the hardware's). One accumulator of 128 tokens x 256 experts in tensor memory; TMA brings one
  // [128 x 64] slab of x and one [256 x 64] slab of W_r per stage, both in the 128-byte swizzle.
  const bool gemv = !PAIR && p.logits_out != nullptr;  // the pair build keeps every tcgen05 instruction at cta_group::2
  if (gemv) {
    if (tid == 0) {
      for (int s = 0; s < RS; ++s) { mbar_init(&S.rfull[s], 1); mbar_init(&S.rempty[s], 1); }
      mbar_init(&S.racc_full, 1);
      mbar_init(&S.racc_empty, N_EPI / 32);
      mbar_init_fence();
    }
    if (warp == WARP_MMA) {
      tmem_alloc(&S.tmem_base, TMEM_COLS);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_r = S.tmem_base;
    const int c0 = min(T, bid * NWARPS * tok_per_warp);
    const int c1 = min(T, c0 + NWARPS * tok_per_warp);
    const int n_rt = (c1 - c0 + TILE_M - 1) / TILE_M;
    if (warp == WARP_TMA) {
      if (lane == 0) {
        tma_prefetch_desc(&p.tm_x);
        tma_prefetch_desc(&p.tm_rw);
        uint32_t n = 0;
        bool ok = true;
        for (int rt = 0; rt < n_rt && ok; ++rt) {
          for (int ks = 0; ks < RK; ++ks, ++n) {
            const uint32_t st = n % RS;
            if (!mbar_wait(&S.rempty[st], ((n / RS) & 1u) ^ 1u, wc, kSiteRouterEmpty)) { ok = false; break; }
            mbar_arrive_expect_tx(&S.rfull[st], A_STAGE_BYTES + B_STAGE_BYTES);
            tma_load_2d(&p.tm_x, static_cast<uint32_t>(ks * 64), static_cast<uint32_t>(c0 + rt * TILE_M),
                        a_ring + st * A_STAGE_BYTES, &S.rfull[st]);
            tma_load_2d(&p.tm_rw, static_cast<uint32_t>(ks * 64), 0u, b_ring + st * B_STAGE_BYTES, &S.rfull[st]);
          }
        }
      }
    } else if (warp == WARP_MMA) {
      if (lane == 0) {
        const uint32_t a_u32 = smem_u32(a_ring), b_u32 = smem_u32(b_ring);
        uint32_t n = 0;
        bool ok = true;
        for (int rt = 0; rt < n_rt && ok; ++rt) {
          if (!mbar_wait(&S.racc_empty, (static_cast<uint32_t>(rt) & 1u) ^ 1u, wc, kSiteRouterAccEmpty)) break;
          tc_fence_after();
          for (int ks = 0; ks < RK; ++ks, ++n) {
            const uint32_t st = n % RS;
            if (!mbar_wait(&S.rfull[st], (n / RS) & 1u, wc, kSiteRouterFull)) { ok = false; break; }
            tc_fence_after();
            const uint64_t da = umma_desc_sw128(a_u32 + st * A_STAGE_BYTES);
            const uint64_t db = umma_desc_sw128(b_u32 + st * B_STAGE_BYTES);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_bf16(tmem_r, da + 2u * k, db + 2u * k, IDESC_ROUTER, (ks | k) ? 1u : 0u);
            umma_commit(&S.rempty[st]);
          }
          if (ok) umma_commit(&S.racc_full);
        }
      }
    } else if (warp >= 4) {
      const int et = tid - 128;
      const int h = et >> 7;        // which 128 experts (EPI_WGS == 2), or which 64 (EPI_WGS == 4)
      const int q = warp & 3;
      const int r = q * 32 + lane;
      constexpr int RCOLS = E / EPI_WGS;
      const uint32_t t_lane = tmem_r + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(h * RCOLS);
      for (int rt = 0; rt < n_rt; ++rt) {
        if (!mbar_wait(&S.racc_full, static_cast<uint32_t>(rt) & 1u, wc, kSiteRouterAccFull)) break;
        tc_fence_after();
        const int row = c0 + rt * TILE_M + r;
#pragma unroll
        for (int c = 0; c < RCOLS / 32; ++c) {
          uint32_t v[32];
          tmem_ld_n<32>(t_lane + c * 32, v);
          tmem_ld_wait();
          if (row < c1) {
            float* dst = p.logits_out + static_cast<size_t>(row) * E + h * RCOLS + c * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t w8[8] = {v[8 * i], v[8 * i + 1], v[8 * i + 2], v[8 * i + 3],
                                      v[8 * i + 4], v[8 * i + 5], v[8 * i + 6], v[8 * i + 7]};
              st_global_256(dst + 8 * i, w8);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.racc_empty);
      }
    }
    // the logits this CTA wrote are read back by its own warps below; the operand rings are reused
    tc_fence_before();
    __syncthreads();
    if (bid == 0 && tid == 0) ws->phase_ns[5] = globaltimer_ns();
  }
  const float* lg_src = gemv ? p.logits_out : p.logits;

  // ================================================================ phase 0
  for (int i = tid; i < NWARPS * E; i += BLOCK) hist[i] = 0;
  __syncthreads();

  // Every warp routes AND quantises its own tokens, one at a time: the first piece of the token's
  // activations is requested before the routing arithmetic (a chain of warp shuffles that leaves most issue
  // slots empty) and consumed after it, so the memory latency of the quantiser hides behind the router.
  // (Splitting the warps into routers and quantisers was measured and is slower: routing wants all twelve.)

  constexpr int NT = 1;  // tokens routed side by side by one warp (two were measured: 8 % slower, the second token's state costs more than the filled latency gains)
  float lg_next[NT][8];
  PROF_DECL(p0_route); PROF_DECL(p0_quant);
  if (t_begin < t_end) {
#pragma unroll
    for (int a = 0; a < NT; ++a) {
      const int tt = min(t_begin + a, t_end - 1);  // an odd tail routes its last token twice and drops the copy
#pragma unroll
      for (int j = 0; j < 8; ++j) lg_next[a][j] = lg_src[static_cast<size_t>(tt) * E + lane + 32 * j];
    }
  }
  for (int t = t_begin; t < t_end; t += NT) {
    int my_id[NT];
    float my_w[NT];
    float lg[NT][8];
    uint4 qraw[NT][QU];
#pragma unroll
    for (int a = 0; a < NT; ++a) {
#pragma unroll
      for (int j = 0; j < 8; ++j) lg[a][j] = lg_next[a][j];
    }
    if (t + NT < t_end) {  // the next tokens' logits are in flight while these are routed
#pragma unroll
      for (int a = 0; a < NT; ++a) {
        const int tt = min(t + NT + a, t_end - 1);
#pragma unroll
        for (int j = 0; j < 8; ++j) lg_next[a][j] = lg_src[static_cast<size_t>(tt) * E + lane + 32 * j];
      }
    }
#pragma unroll
    for (int a = 0; a < NT; ++a)
      if (t + a < t_end) quant_token_load(p, t + a, 0, lane, qraw[a]);
    { PROF_T0();
    route_tokens<NT>(lg, p.router_bias, lane, my_id, my_w);
    PROF_ADD(p0_route); }
    PROF_T0();
#pragma unroll
    for (int a = 0; a < NT; ++a) {
      if (t + a >= t_end) break;
      if (lane < TOP_K) {
        int lid = my_id[a];
        if constexpr (EP_BUILD) lid = (my_id[a] >= 0) ? p.expert_map[my_id[a]] : -1;
        if (lid >= E_LOCAL) lid = -1;
        p.topk_ids[(t + a) * TOP_K + lane] = lid;
        p.topk_weights[(t + a) * TOP_K + lane] = my_w[a];
        if (lid >= 0) hist[warp * E + lid] += 1;  // ids of one token are distinct: no conflict
      }
      __syncwarp();  // the next token's increments may hit the same counters from other lanes
      float gdot = 0.f;
      if (p.sh_gate == nullptr) {
        quant_token_store<false>(p, t + a, 0, lane, qraw[a], nullptr, gdot);
#pragma unroll 1
        for (int piece = 1; piece < Q_PIECES; ++piece) {
          quant_token_load(p, t + a, piece, lane, qraw[a]);
          quant_token_store<false>(p, t + a, piece, lane, qraw[a], nullptr, gdot);
        }
      } else {   // gate of the shared expert: sigmoid(x . g), one value per token
        quant_token_store<true>(p, t + a, 0, lane, qraw[a], p.sh_gate, gdot);
#pragma unroll 1
        for (int piece = 1; piece < Q_PIECES; ++piece) {
          quant_token_load(p, t + a, piece, lane, qraw[a]);
          quant_token_store<true>(p, t + a, piece, lane, qraw[a], p.sh_gate, gdot);
        }
        gdot = warp_sum_f(gdot);
        if (lane == 0) p.sh_gate_w[t + a] = det_sigmoidf(gdot);
      }
    }
    __syncwarp();
    PROF_ADD(p0_quant);
  }
  if (tid == 0) { PROF_STORE(7, p0_route); PROF_STORE(15, p0_quant); }
  __syncthreads();
  if (tid < E) {
    int c = 0;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) c += hist[w * E + tid];
    ws->cta_hist[bid][tid] = c;
  }

  bool alive = grid_sync(wc, 0, &S.flag);
  if (bid == 0 && tid == 0) ws->phase_ns[1] = globaltimer_ns();

  // ================================================================ phase 1
  // Scheduling unit: a tile of 128 sorted rows on one CTA, or a pair of them on a cluster of two CTAs.
  constexpr int SCHED_ROWS = PAIR ? 2 * TILE_M : TILE_M;
  constexpr int SCHED_UNITS = PAIR ? kGrid / 2 : kGrid;
  const int sched_me = PAIR ? (bid >> 1) : bid;
  if (alive) {
    if (tid < E) { ph1_tot[tid] = 0; ph1_pre[tid] = 0; }
    __syncthreads();
    {
      // 64 column groups of 4 experts x BLOCK/64 row groups of CTAs
      const int col = tid & 63, rg = tid >> 6;
      int4 tot = make_int4(0, 0, 0, 0), pre = make_int4(0, 0, 0, 0);
#pragma unroll 5
      for (int b = rg; b < kGrid; b += BLOCK / 64) {
        const int4 c = __ldcg(reinterpret_cast<const int4*>(&ws->cta_hist[b][col * 4]));
        tot.x += c.x; tot.y += c.y; tot.z += c.z; tot.w += c.w;
        if (b < bid) { pre.x += c.x; pre.y += c.y; pre.z += c.z; pre.w += c.w; }
      }
      atomicAdd(&ph1_tot[col * 4 + 0], tot.x); atomicAdd(&ph1_tot[col * 4 + 1], tot.y);
      atomicAdd(&ph1_tot[col * 4 + 2], tot.z); atomicAdd(&ph1_tot[col * 4 + 3], tot.w);
      atomicAdd(&ph1_pre[col * 4 + 0], pre.x); atomicAdd(&ph1_pre[col * 4 + 1], pre.y);
      atomicAdd(&ph1_pre[col * 4 + 2], pre.z); atomicAdd(&ph1_pre[col * 4 + 3], pre.w);
    }
    __syncthreads();
    int cnt = 0, tiles_e = 0;
    if (tid < E) {
      cnt = ph1_tot[tid];
      tiles_e = (cnt + SCHED_ROWS - 1) / SCHED_ROWS * NCH;  // units of work: (tile, chunk), chunk fastest
      scan_cnt[tid] = cnt;
      scan_tile[tid] = tiles_e;
    }
    __syncthreads();
    for (int d = 1; d < E; d <<= 1) {
      int vc = 0, vt = 0;
      if (tid < E && tid >= d) { vc = scan_cnt[tid - d]; vt = scan_tile[tid - d]; }
      __syncthreads();
      if (tid < E) { scan_cnt[tid] += vc; scan_tile[tid] += vt; }
      __syncthreads();
    }
    if (tid < E) {
      const int off_e = scan_cnt[tid] - cnt;
      const int tbase = scan_tile[tid] - tiles_e;
      if (tid == E - 1) S.total_tiles = tbase + tiles_e;
      if (bid == 0) {
        ws->expert_counts[tid] = cnt;
        ws->expert_offsets[tid] = off_e;
        if (tid == E - 1) {
          ws->expert_offsets[E] = off_e + cnt;
          ws->total_tiles = tbase + tiles_e;
        }
      }
      for (int i = 0; i < tiles_e; ++i) {
        const int g = tbase + i;
        if (g % SCHED_UNITS == sched_me) {
          const int slot = g / SCHED_UNITS;
          if (slot < MAX_MY_TILES) {
            TileInfo ti;
            ti.e = tid;
            // pair schedule: rank 0 of the cluster takes the first 128 rows of the 256, rank 1 the rest (maybe none)
            ti.row0 = off_e + (i / NCH) * SCHED_ROWS + (PAIR ? (bid & 1) * TILE_M : 0);
            ti.rows = max(0, min(TILE_M, off_e + cnt - ti.row0));
            ti.chunk = i % NCH;
            S.tiles[slot] = ti;
          } else {
            report_error(ws, kErrBounds, 1, static_cast<uint32_t>(g), static_cast<uint32_t>(slot));
          }
        }
      }
      // turn the per-warp histograms into per-warp write cursors
      int base = off_e + ph1_pre[tid];
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) {
        const int h = hist[w * E + tid];
        hist[w * E + tid] = base;
        base += h;
      }
    }
    __syncthreads();
    // the shared expert's units follow the routed ones in the deal: token tile j (128 tokens), chunk fastest
    int sh_units = 0;
    if (p.sh_on) {
      const int tok_tiles = (T + TILE_M - 1) / TILE_M;
      const int mine = (tok_tiles > p.sh_part) ? (tok_tiles - p.sh_part + p.sh_parts - 1) / p.sh_parts : 0;
      sh_units = mine * NCH;
      const int tt_routed = S.total_tiles;
      for (int i = tid; i < sh_units; i += BLOCK) {
        const int g = tt_routed + i;
        if (g % SCHED_UNITS == sched_me) {
          const int slot = g / SCHED_UNITS;
          if (slot < MAX_MY_TILES) {
            TileInfo ti;
            ti.e = SHARED_E;
            ti.row0 = (p.sh_part + (i / NCH) * p.sh_parts) * TILE_M;
            ti.rows = max(0, min(TILE_M, T - ti.row0));
            ti.chunk = i % NCH;
            S.tiles[slot] = ti;
          } else {
            report_error(ws, kErrBounds, 3, static_cast<uint32_t>(g), static_cast<uint32_t>(slot));
          }
        }
      }
    }
    if (tid == 0) {
      const int tt = S.total_tiles + sh_units;
      S.n_my_tiles = (tt > sched_me) ? min(MAX_MY_TILES, (tt - sched_me + SCHED_UNITS - 1) / SCHED_UNITS) : 0;
    }
    // stable scatter: each warp re-walks its own tokens in ascending order
    for (int t = t_begin; t < t_end; ++t) {
      if (lane < TOP_K) {
        const int lid = p.topk_ids[t * TOP_K + lane];
        if (lid >= 0) {
          const int pos = hist[warp * E + lid]++;
          if (pos >= 0 && pos < numel) p.sorted_ids[pos] = t * TOP_K + lane;
          else report_error(ws, kErrBounds, 2, static_cast<uint32_t>(pos), static_cast<uint32_t>(t));
        }
      }
      __syncwarp();
    }
  }

  alive = grid_sync(wc, 1, &S.flag) && alive;
  if (bid == 0 && tid == 0) ws->phase_ns[2] = globaltimer_ns();
  // phase 1 wrote the operand rings with ordinary stores (histograms, scan arrays); phase 2 fills them through
  // the async proxy (TMA), so order the two proxies once here
  fence_proxy_async_smem();

  // ================================================================ phase 2
  // Pair build: the MMA thread lives in the cluster's rank-0 CTA ("leader"). Its fullA barrier also
  // receives one forwarded arrival per stage for the peer's gathered rows, and its tmem_empty /
  // inter_ready barriers collect the epilogue warps of both CTAs.
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = crank == 0u;
  if (tid == 0) {
    const uint32_t both = PAIR ? 2u : 1u;
    for (int s = 0; s < SA; ++s) {
      mbar_init(&S.fullA[s], N_GATHER + ((PAIR && leader) ? 1u : 0u));
      mbar_init(&S.emptyA[s], 1);
    }
    for (int s = 0; s < SB; ++s) { mbar_init(&S.fullB[s], 1); mbar_init(&S.emptyB[s], 1); }
    for (int s = 0; s < NBUF; ++s) { mbar_init(&S.tmem_full[s], 1); mbar_init(&S.tmem_empty[s], both * (N_EPI / 32)); }
#ifdef MONO_PROFILE
    for (int i = 0; i < 48; ++i) (&S.whist[0][0])[i] = 0ull;
#endif
    for (int s = 0; s < NP; ++s) mbar_init(&S.inter_ready[s], both * (N_EPI / 32));
    mbar_init_fence();
  }
  if (warp == WARP_MMA && !gemv) {  // phase R already holds the allocation
    if constexpr (PAIR) {
      tmem_alloc_pair(&S.tmem_base, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&S.tmem_base, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  else __syncthreads();
  tc_fence_after();
  // cluster address of the leader's copy of a barrier of the shared state (both CTAs signal it)
  const uint32_t s_local = smem_u32(&S);
  const uint32_t s_leader = PAIR ? map_to_cta(s_local, 0) : s_local;
  auto at_leader = [&](const uint64_t* bar) -> uint32_t { return s_leader + (smem_u32(bar) - s_local); };
  const uint32_t tmem_base = S.tmem_base;
  const int n_my = alive ? S.n_my_tiles : 0;

  if (warp < 4) {
    reg_dec<REGS_PRODUCER>();
    if (warp == WARP_TMA) {
      // ---------------------------------------------------------- weight producer
      if (lane == 0) {
        tma_prefetch_desc(&p.tm_up);
        tma_prefetch_desc(&p.tm_down);
        uint32_t nb = 0;
        bool ok = true;
        PROF_DECL(pw_emptyB);
        for (int it = 0; it < ((MONO_ABLATE & 64) ? 0 : n_my) && ok; ++it) {
          const int ch = S.tiles[it].chunk;
          const bool sh = S.tiles[it].e == SHARED_E;
          const int e = sh ? 0 : S.tiles[it].e;                     // row base inside the weight tensor
          const CUtensorMap* map_up = sh ? &p.tm_sh_up : &p.tm_up;
          const CUtensorMap* map_down = sh ? &p.tm_sh_down : &p.tm_down;
          for (int ps = 0; ps < NP && ok; ++ps) {
            const uint32_t yg = static_cast<uint32_t>(e * N_UP + ch * CHUNK_COLS + ps * 128);
            const uint32_t yu = yg + N_HALF;
            for (int ks = 0; ks < NK; ++ks) {
              const uint32_t st = nb % SB, ph = (nb / SB) & 1u;
              { PROF_T0();
              if (!mbar_wait(&S.emptyB[st], ph ^ 1u, wc, kSiteEmptyB)) { ok = false; break; }
              PROF_ADD(pw_emptyB); }
              uint8_t* dst = b_ring + st * B_STAGE_BYTES;
              const uint32_t x = static_cast<uint32_t>(ks * 128);
              if constexpr (PAIR) {
                // this CTA's half of the stage: the rows the non-pair layout gives to warpgroup `crank`
                // (HCB gate columns, then the HCB matching up columns); the bytes of both halves are
                // counted on the leader's barrier
                if (leader) mbar_arrive_expect_tx(&S.fullB[st], 2 * B_STAGE_BYTES);
                const uint32_t co = crank * HCB;
                tma_load_2d_pair(map_up, x, yg + co, dst, at_leader(&S.fullB[st]));
                tma_load_2d_pair(map_up, x, yu + co, dst + HCB * 128, at_leader(&S.fullB[st]));
                ++nb;
                continue;
              }
              mbar_arrive_expect_tx(&S.fullB[st], (MONO_ABLATE & 16) ? 0 : B_STAGE_BYTES);
              if constexpr ((MONO_ABLATE & 16) != 0) { ++nb; continue; }
              // shared rows of buffer j, warpgroup h: [j*BC + h*WC, +HCB) gate columns c + j*PASS_STRIDE + h*HCB ..,
              // then the HCB matching up columns
#pragma unroll
              for (int j = 0; j < NSPLIT; ++j) {
#pragma unroll
                for (int hh = 0; hh < EPI_WGS; ++hh) {
                  const uint32_t co = static_cast<uint32_t>(j * PASS_STRIDE + hh * HCB);
                  tma_load_2d(map_up, x, yg + co, dst + (j * BC + hh * WC) * 128, &S.fullB[st]);
                  tma_load_2d(map_up, x, yu + co, dst + (j * BC + hh * WC + HCB) * 128, &S.fullB[st]);
                }
              }
              ++nb;
            }
          }
          for (int hb = 0; hb < NHB && ok; ++hb) {
            const uint32_t y = static_cast<uint32_t>(e * H_DIM + hb * 256);
            for (int dk = 0; dk < NP; ++dk) {
              const uint32_t st = nb % SB, ph = (nb / SB) & 1u;
              if (!mbar_wait(&S.emptyB[st], ph ^ 1u, wc, kSiteEmptyB)) { ok = false; break; }
              uint8_t* dst = b_ring + st * B_STAGE_BYTES;
              const uint32_t x = static_cast<uint32_t>((ch * NP + dk) * 128);
              if constexpr (PAIR) {
                if (leader) mbar_arrive_expect_tx(&S.fullB[st], 2 * B_STAGE_BYTES);
#pragma unroll
                for (int j = 0; j < B_ROWS / HCB; ++j)
                  tma_load_2d_pair(map_down, x, y + crank * B_ROWS + j * HCB, dst + j * HCB * 128, at_leader(&S.fullB[st]));
                ++nb;
                continue;
              }
              mbar_arrive_expect_tx(&S.fullB[st], (MONO_ABLATE & 16) ? 0 : B_STAGE_BYTES);
              if constexpr ((MONO_ABLATE & 16) != 0) { ++nb; continue; }
#pragma unroll
              for (int j = 0; j < 256 / HCB; ++j) tma_load_2d(map_down, x, y + j * HCB, dst + j * HCB * 128, &S.fullB[st]);
              ++nb;
            }
          }
        }
        PROF_STORE(0, pw_emptyB);
      }
    } else if (warp == WARP_MMA) {
      // ---------------------------------------------------------- MMA issuer
      if (PAIR && !leader) {
        // The peer CTA issues no MMA. Its lane 0 forwards "my gathered rows of this stage have landed"
        // to the leader's barrier (cp.async can only signal a barrier of its own CTA).
        if (lane == 0) {
          uint32_t na = 0;
          bool ok = true;
          for (int it = 0; it < n_my && ok; ++it) {
            for (int s = 0; s < NP * NK; ++s, ++na) {
              const uint32_t sa = na % SA;
              if (!mbar_wait(&S.fullA[sa], (na / SA) & 1u, wc, kSiteFullA)) { ok = false; break; }
              fence_proxy_async_smem();
              mbar_arrive_cluster(at_leader(&S.fullA[sa]));
            }
          }
        }
      } else if (MONO_MMA_WARP != 0 || lane == 0) {
        // MONO_MMA_WARP: the whole warp walks the loop in uniform control flow and waits together; an elected lane
        // issues the tcgen05 instructions. With a single lane in a divergent branch instead, every descriptor and
        // address has to be moved into a uniform register per instruction, and the seven tcgen05 instructions of a
        // slab step then take longer to issue than the tensor core takes to execute them.
        auto wait_bar = [&](uint64_t* bar, uint32_t parity, uint32_t site) -> bool {
          if constexpr (MONO_MMA_WARP != 0) return mbar_wait_warp(bar, parity, wc, site);
          else return mbar_wait(bar, parity, wc, site);
        };
        auto issuer = [&]() -> bool {
          if constexpr (MONO_MMA_WARP != 0) return elect_one_sync();
          else return true;
        };
        uint32_t nb = 0, na = 0, nt = 0;
        bool ok = true;
#if defined(MONO_TRACE) && defined(MONO_PROFILE)
        int tr_m = 0;
#endif
        PROF_DECL(pm_fullB); PROF_DECL(pm_fullA); PROF_DECL(pm_tmem); PROF_DECL(pm_inter); PROF_DECL(pm_total);
#ifdef MONO_PROFILE
        const long long pm_start = clock64();
#endif
        const uint32_t a_ring_u32 = smem_u32(a_ring), b_ring_u32 = smem_u32(b_ring), inter_u32 = smem_u32(inter);
        for (int it = 0; it < n_my && ok; ++it) {
          for (int s = 0; s < NP * NK; ++s) {
            const uint32_t sb = nb % SB, sa = na % SA;
            TRACE_M(0);
            { PROF_T0();
            if ((MONO_ABLATE & 64) == 0 && !wait_bar(&S.fullB[sb], (nb / SB) & 1u, kSiteFullB)) { ok = false; break; }
            PROF_ADD(pm_fullB); }
            TRACE_M(1);
            { PROF_T0();
            if ((MONO_ABLATE & 64) == 0 && !wait_bar(&S.fullA[sa], (na / SA) & 1u, kSiteFullA)) { ok = false; break; }
            PROF_ADD(pm_fullA); }
            TRACE_M(2);
            // the gathered rows were written by cp.async (generic proxy); the tensor core reads them through the async proxy
            fence_proxy_async_smem();
            const uint64_t da = umma_desc_sw128(a_ring_u32 + sa * A_STAGE_BYTES);
#pragma unroll
            for (int j = 0; j < NSPLIT; ++j) {
              const uint32_t buf = nt % NBUF;
              { PROF_T0();
              if (!wait_bar(&S.tmem_empty[buf], ((nt / NBUF) & 1u) ^ 1u, kSiteTmemEmpty)) { ok = false; break; }
              PROF_ADD(pm_tmem); PROF_HIST(1, ((s % NK) < 16 ? (s % NK) : 15), lane == 0); }
              TRACE_M(3);
              tc_fence_after();
              const uint64_t db = umma_desc_sw128(b_ring_u32 + sb * B_STAGE_BYTES + j * BC * 128);
              const uint32_t d = tmem_base + buf * BC;
              if (issuer()) {
                if constexpr (PAIR) {
#pragma unroll
                  for (int k = 0; k < 4; ++k) umma_f8_pair(d, da + 2u * k, db + 2u * k, IDESC, k > 0 ? 1u : 0u);
                  umma_commit_pair(&S.tmem_full[buf]);
                } else {
#pragma unroll
                  for (int k = 0; k < ((MONO_ABLATE & 128) ? 8 : 4); ++k) umma_f8(d, da + 2u * (k & 3), db + 2u * (k & 3), IDESC, k > 0 ? 1u : 0u);
                  umma_commit(&S.tmem_full[buf]);
                }
              }
              if constexpr (MONO_MMA_WARP != 0) __syncwarp();
              ++nt;
            }
            if (!ok) break;
            if ((MONO_ABLATE & 64) == 0 && issuer()) {
              if constexpr (PAIR) { umma_commit_pair(&S.emptyA[sa]); umma_commit_pair(&S.emptyB[sb]); }
              else { umma_commit(&S.emptyA[sa]); umma_commit(&S.emptyB[sb]); }
            }
            if constexpr (MONO_MMA_WARP != 0) __syncwarp();
            ++nb; ++na;
            TRACE_M(4);
          }
          if (!ok) break;
          for (int s = 0; s < NHB * NP; ++s) {
            const int dk = s % NP;
            const uint32_t sb = nb % SB;
            if (s < NP) {
              // K slab dk of the down projection reads the 128 intermediate columns pass dk wrote: the first
              // slabs start while the epilogue is still in the SiLU section of the last pass
              { PROF_T0();
              if (!wait_bar(&S.inter_ready[dk], static_cast<uint32_t>(it) & 1u, kSiteInterReady)) { ok = false; break; }
              PROF_ADD(pm_inter); }
              tc_fence_after();
            }
            TRACE_M(0);
            { PROF_T0();
            if ((MONO_ABLATE & 64) == 0 && !wait_bar(&S.fullB[sb], (nb / SB) & 1u, kSiteFullB)) { ok = false; break; }
            PROF_ADD(pm_fullB); }
            TRACE_M(1);
            TRACE_M(2);
            const uint64_t da = umma_desc_sw128(inter_u32 + (dk % INTER_SLOTS) * A_STAGE_BYTES);
#pragma unroll
            for (int j = 0; j < NSPLIT; ++j) {
              const uint32_t buf = nt % NBUF;
              { PROF_T0();
              if (!wait_bar(&S.tmem_empty[buf], ((nt / NBUF) & 1u) ^ 1u, kSiteTmemEmpty)) { ok = false; break; }
              PROF_ADD(pm_tmem); PROF_HIST(1, 16 + dk, lane == 0); }
              TRACE_M(3);
              tc_fence_after();
              const uint64_t db = umma_desc_sw128(b_ring_u32 + sb * B_STAGE_BYTES + j * BC * 128);
              const uint32_t d = tmem_base + buf * BC;
              if (issuer()) {
                if constexpr (PAIR) {
#pragma unroll
                  for (int k = 0; k < 4; ++k) umma_f8_pair(d, da + 2u * k, db + 2u * k, IDESC, k > 0 ? 1u : 0u);
                  umma_commit_pair(&S.tmem_full[buf]);
                } else {
#pragma unroll
                  for (int k = 0; k < ((MONO_ABLATE & 128) ? 8 : 4); ++k) umma_f8(d, da + 2u * (k & 3), db + 2u * (k & 3), IDESC, k > 0 ? 1u : 0u);
                  umma_commit(&S.tmem_full[buf]);
                }
              }
              if constexpr (MONO_MMA_WARP != 0) __syncwarp();
              ++nt;
            }
            if (!ok) break;
            if ((MONO_ABLATE & 64) == 0 && issuer()) { if constexpr (PAIR) umma_commit_pair(&S.emptyB[sb]); else umma_commit(&S.emptyB[sb]); }
            if constexpr (MONO_MMA_WARP != 0) __syncwarp();
            ++nb;
            TRACE_M(4);
          }
        }
#ifdef MONO_PROFILE
        pm_total = clock64() - pm_start;
#endif
        if (lane == 0) {
          PROF_STORE(1, pm_fullB); PROF_STORE(2, pm_fullA); PROF_STORE(3, pm_tmem); PROF_STORE(4, pm_inter);
          PROF_STORE(5, pm_total);
        }
#if defined(MONO_PROFILE) && !defined(MONO_TRACE)
        if (lane == 0) for (int i = 0; i < 24; ++i) p.ws->prof[blockIdx.x][40 + i] = S.whist[1][i];
#endif
      }
    } else {
      // ---------------------------------------------------------- activation gather (warps 2-3, 64 threads)
      // cp.async 16 B with the 128-byte swizzle applied by hand.
      // (TMA tile::gather4 was measured here as well: correct, but a third slower than this path
      // because every gathered row is a separate 128-byte request.)
      const int gt = tid - WARP_GATHER0 * 32;
      // Eight neighbouring lanes copy the eight 16-byte pieces of ONE row, so a warp instruction touches
      // 4 whole lines of global memory and 512 contiguous bytes of shared memory (one row per lane would be
      // 32 lines per instruction and a 4-way bank conflict). Thread g: piece g % 8 of rows g / 8 + 8 i.
      const int gc = gt & 7, gr = gt >> 3;
      constexpr int ROWS_PER_THREAD = TILE_M / 8;
      uint32_t na = 0;
      bool dead = false;  // after an abort: keep the loop structure (the named barrier stays matched), skip the work
      PROF_DECL(pg_emptyA);
      const uint32_t a_ring_u32 = smem_u32(a_ring);
      for (int it = 0; it < ((MONO_ABLATE & 64) ? 0 : n_my); ++it) {
        const TileInfo ti = S.tiles[it];
        // the tile's 128 source tokens go through shared memory (two rows looked up per thread); the two
        // buffers alternate by tile, and the barrier of tile it+1 separates the last read of tile it-1's
        // buffer from its next fill
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = gt + hh * 64;
          int t = -1;
          if (r < ti.rows) {
            if (ti.e == SHARED_E) {
              t = ti.row0 + r;                       // the shared expert takes the tokens in order
            } else {
              const int fi = __ldcg(&p.sorted_ids[ti.row0 + r]);
              if (fi >= 0 && fi < numel) t = fi / TOP_K;
            }
          }
          S.gather_tok[it & 1][r & 7][r >> 3] = t;
        }
        named_bar_sync(2, N_GATHER);
        for (int s = 0; s < NP * NK; ++s) {
          const int ks = s % NK;
          const uint32_t sa = na % SA;
          { PROF_T0();
          if (!dead && !mbar_wait(&S.emptyA[sa], ((na / SA) & 1u) ^ 1u, wc, kSiteEmptyA)) dead = true;
          PROF_ADD(pg_emptyA); }
          if (dead) continue;
          // row gr + 8 i sits in eight-row group i (1024 bytes each) at row position gr, piece gc ^ gr
          const uint32_t dst = a_ring_u32 + sa * A_STAGE_BYTES + gr * 128 + ((gc ^ gr) << 4);
          const uint8_t* g0 = p.act_fp8 + ks * 128 + gc * 16;
          if constexpr ((MONO_ABLATE & 8) == 0) {
#pragma unroll
            for (int i4 = 0; i4 < ROWS_PER_THREAD / 4; ++i4) {
              const int4 t4 = *reinterpret_cast<const int4*>(&S.gather_tok[it & 1][gr][4 * i4]);
              const int tok[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (tok[i] >= 0) cp_async16(dst + (4 * i4 + i) * 1024, g0 + static_cast<size_t>(tok[i]) * K_DIM);
            }
          }
          // the barrier receives this thread's arrival when the copies above have landed
          cp_async_arrive_noinc(&S.fullA[sa]);
          ++na;
        }
      }
      cp_async_commit();
      cp_async_wait<0>();
      if (gt == 0) { PROF_STORE(6, pg_emptyA); }
    }
  } else {
    // ------------------------------------------------------------ epilogue (EPI_WGS x 128 threads)
    reg_inc<REGS_EPILOGUE>();
    {
      const int et = tid - 128;
      const int h = et >> 7;               // warpgroup: which WC columns of every accumulator buffer
      const int q = warp & 3;              // TMEM lane quarter this warp may read
      const int r = q * 32 + lane;         // row of the tile
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(h * WC);
      uint32_t nt = 0;
      bool dead = false;  // after an abort: keep the loop structure (named barriers stay matched), skip the work
      // Accumulators, pairs of adjacent columns. Buffer j of a slab owns acc[j*WC/2, (j+1)*WC/2):
      // first the HCB gate columns (down projection: the first half of WC output columns), then the up columns.
      float2 acc[TCOLS / 2];
#if defined(MONO_TRACE) && defined(MONO_PROFILE)
      int tr_e = 4000;
#endif
      PROF_DECL(pe_bar); PROF_DECL(pe_zero); PROF_DECL(pe_wait); PROF_DECL(pe_up); PROF_DECL(pe_silu); PROF_DECL(pe_down); PROF_DECL(pe_store);
#ifdef MONO_PROFILE
      const long long pe_start = clock64();
#endif

      // Read one accumulator buffer out of tensor memory and fold it into part j of the register
      // accumulators: acc += D * scale (s_lo for the first HCB columns, s_hi for the rest). The
      // buffer goes back to the MMA thread as soon as its contents are in registers.
      auto promote = [&](int j, uint32_t buf, float s_lo, float s_hi) {
        tc_fence_after();
        if constexpr ((MONO_ABLATE & 1) != 0) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { if (PAIR && !leader) mbar_arrive_cluster(at_leader(&S.tmem_empty[buf])); else mbar_arrive(&S.tmem_empty[buf]); }
          return;
        }
#pragma unroll
        for (int c = 0; c < NLD; ++c) {
          uint32_t v[LDW];
          tmem_ld_n<LDW>(t_lane + buf * BC + c * LDW, v);
          tmem_ld_wait();
          if (c == NLD - 1) {
            // one arrival per warp: per-thread arrivals on one shared-memory word serialise
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (PAIR && !leader) mbar_arrive_cluster(at_leader(&S.tmem_empty[buf])); else mbar_arrive(&S.tmem_empty[buf]); }
            TRACE_E(2);
          }
#pragma unroll
          for (int i = 0; i < LDW / 2; ++i) {
            const int pair = c * (LDW / 2) + i;              // pair of columns inside this warpgroup's WC
            const float sc = (pair < HCB / 2) ? s_lo : s_hi;
            acc[j * (WC / 2) + pair] = __ffma2_rn(make_float2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])),
                                                  make_float2(sc, sc), acc[j * (WC / 2) + pair]);
          }
        }
      };

      // Scales are staged in shared memory one tile ahead: nothing in the slab loop waits on a
      // global load. stage_* below fetch tile `nx`: its row's slot id, routing weight and
      // activation scales (warpgroups 0 and 1 load half a row each), and the expert's weight
      // scales (into buffer nx & 1).
      // nfi: index of the row's partial row (routed: its flat slot t * top_k + k; shared expert: numel + token);
      // ntok: its token
      int nfi = -1, ntok = -1;
      float nrw = 0.f, wsu_v = 0.f, wsd_v = 0.f;
      float4 as_v = make_float4(0.f, 0.f, 0.f, 0.f);
      auto stage_ids = [&](int nx) {
        const TileInfo tn = S.tiles[nx];
        const bool sh = tn.e == SHARED_E;
        nfi = -1;
        ntok = -1;
        if (r < tn.rows) {
          if (sh) {
            ntok = tn.row0 + r;
            nfi = numel + ntok;
          } else {
            nfi = __ldcg(&p.sorted_ids[tn.row0 + r]);
            if (nfi < 0 || nfi >= numel) nfi = -1;
            else ntok = nfi / TOP_K;
          }
        }
        const float* su = sh ? p.sh_up_scales : p.up_w_scales;
        const float* sd = sh ? p.sh_down_scales : p.down_w_scales;
        const int es = sh ? 0 : tn.e;
        if (et < WSU_N) wsu_v = __ldg(su + wsu_index(es, tn.chunk, et));
        if (et < WSD_N) wsd_v = __ldg(sd + wsd_index(es, tn.chunk, et));
      };
      auto stage_weight_store = [&](int nx) {
        const bool sh = S.tiles[nx].e == SHARED_E;
        if (nfi < 0) nrw = 0.f;
        else if (!sh) nrw = __ldcg(&p.topk_weights[nfi]);
        else nrw = (p.sh_gate != nullptr) ? __ldcg(&p.sh_gate_w[ntok]) : 1.f;
        if (et < WSU_N) wsu_sm[(nx & 1) * WSU_N + et] = wsu_v;
        if (et < WSD_N) wsd_sm[(nx & 1) * WSD_N + et] = wsd_v;
        const float* su = sh ? p.sh_up_scales : p.up_w_scales;
        const float* sd = sh ? p.sh_down_scales : p.down_w_scales;
        const int es = sh ? 0 : S.tiles[nx].e;
        if constexpr (WSU_N > N_EPI) {
          for (int i = et + N_EPI; i < WSU_N; i += N_EPI)
            wsu_sm[(nx & 1) * WSU_N + i] = __ldg(su + wsu_index(es, S.tiles[nx].chunk, i));
        }
        if constexpr (WSD_N > N_EPI) {
          for (int i = et + N_EPI; i < WSD_N; i += N_EPI)
            wsd_sm[(nx & 1) * WSD_N + i] = __ldg(sd + wsd_index(es, S.tiles[nx].chunk, i));
        }
      };
      auto as_piece_load = [&](int j) {
        as_v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (h < 2 && nfi >= 0)
          as_v = __ldcg(reinterpret_cast<const float4*>(p.act_scales + static_cast<size_t>(ntok) * NK + h * (NK / 2) + 4 * j));
      };
      auto as_piece_store = [&](int j) {
        if (h < 2) {
          float* d = as_sm + (h * (NK / 2) + 4 * j) * TILE_M + r;
          d[0] = as_v.x; d[TILE_M] = as_v.y; d[2 * TILE_M] = as_v.z; d[3 * TILE_M] = as_v.w;
        }
      };
      if (n_my > 0) {
        stage_ids(0);
        stage_weight_store(0);
        for (int j = 0; j < AS_PIECES; ++j) { as_piece_load(j); as_piece_store(j); }
      }

      for (int it = 0; it < n_my; ++it) {
        const TileInfo ti = S.tiles[it];
        const int fi = nfi;
        const float rw = nrw;
        const float2 rw2 = make_float2(rw, rw);
        const float* wsu_t = wsu_sm + (it & 1) * WSU_N;
        const float* wsd_t = wsd_sm + (it & 1) * WSD_N;
        const bool has_next = it + 1 < n_my;
        float iscale[NP];
        { PROF_T0();
        named_bar_sync(1, N_EPI);  // this tile's staged scales are visible to all epilogue threads
        PROF_ADD(pe_bar); }

        // ---------------- up projection + SiLU*mul + requantisation
        for (int ps = 0; ps < NP; ++ps) {
          { PROF_T0();
#pragma unroll
          for (int i = 0; i < TCOLS / 2; ++i) acc[i] = make_float2(0.f, 0.f);
          PROF_ADD(pe_zero); }
          for (int ks = 0; ks < NK; ++ks) {
            const float a_s = as_sm[ks * TILE_M + r];
            const float s_g = __fmul_rn(wsu_t[ps * NK + ks], a_s), s_u = __fmul_rn(wsu_t[(NP + ps) * NK + ks], a_s);
#pragma unroll
            for (int j = 0; j < NSPLIT; ++j) {
              const uint32_t buf = nt % NBUF;
              TRACE_E(0);
              { PROF_T0();
              if (!dead && !mbar_wait(&S.tmem_full[buf], (nt / NBUF) & 1u, wc, kSiteTmemFull)) dead = true;
              PROF_ADD(pe_wait); PROF_HIST(0, (ks < 16 ? ks : 15), et == 0); }
              TRACE_E(1);
              PROF_T0();
              if (!dead) promote(j, buf, s_g, s_u);
              PROF_ADD(pe_up);
              TRACE_E(3);
              ++nt;
            }
          }
          PROF_T0();
          if (p.dbg_acc != nullptr && fi >= 0 && !dead && ti.e != SHARED_E) {
            float* d = p.dbg_acc + static_cast<size_t>(ti.row0 + r) * N_UP;
#pragma unroll
            for (int j = 0; j < NSPLIT; ++j) {
              const int col0 = ti.chunk * CHUNK_COLS + ps * 128 + j * PASS_STRIDE + h * HCB;
#pragma unroll
              for (int i = 0; i < HCB / 2; ++i) {
                d[col0 + 2 * i] = acc[j * (WC / 2) + i].x;
                d[col0 + 2 * i + 1] = acc[j * (WC / 2) + i].y;
                d[N_HALF + col0 + 2 * i] = acc[j * (WC / 2) + HCB / 2 + i].x;
                d[N_HALF + col0 + 2 * i + 1] = acc[j * (WC / 2) + HCB / 2 + i].y;
              }
            }
          }
          // SiLU(gate) * up (kernel/qwen_tp/src/prefill_mono_final_nb.cu:678), written over the gate columns
          float mx = 0.f;
#pragma unroll
          for (int j = 0; j < ((MONO_ABLATE & 2) ? 0 : NSPLIT); ++j) {
#pragma unroll
            for (int i = 0; i < HCB / 2; ++i) {
              const float2 g = acc[j * (WC / 2) + i], u = acc[j * (WC / 2) + HCB / 2 + i];
              // the reference's form (exp and division on the special-function unit). A tanh.approx form needs one
              // special-function operation instead of two and is 15 us faster per layer, but its 2^-11 relative error
              // moves enough e4m3 codes of the intermediate to push about one output in 10^5 beyond 2e-2 rms
              const float v0 = __fdividef(u.x * g.x, 1.0f + __expf(-g.x));
              const float v1 = __fdividef(u.y * g.y, 1.0f + __expf(-g.y));
              acc[j * (WC / 2) + i] = make_float2(v0, v1);
              mx = fmaxf(mx, fmaxf(fabsf(v0), fabsf(v1)));
            }
          }
          // the row's amax over the pass's 128 columns: every warpgroup holds NSPLIT*HCB of them
          S.rowmax[ps & 1][h][r] = mx;
          named_bar_sync(1, N_EPI);
#pragma unroll
          for (int hh = 0; hh < EPI_WGS; ++hh) mx = fmaxf(mx, S.rowmax[ps & 1][hh][r]);
          const bool nz = mx > FLT_MIN;
          const float inv = nz ? __fdiv_rn(448.0f, mx) : 0.f;
          const float my_scale = nz ? __fdiv_rn(mx, 448.0f) : (1.0f / 448.0f);
#pragma unroll
          for (int qq = 0; qq < NP; ++qq)
            if (qq == ps) iscale[qq] = my_scale;  // static indexing keeps the array in registers
          uint8_t* irow = inter + (ps % INTER_SLOTS) * A_STAGE_BYTES;
#pragma unroll
          for (int j = 0; j < ((MONO_ABLATE & 2) ? 0 : NSPLIT); ++j) {
#pragma unroll
            for (int c = 0; c < HCB / 16; ++c) {
              const float2* a = &acc[j * (WC / 2) + c * 8];
              uint4 qv;
              qv.x = pack_e4m3x4(a[0].x * inv, a[0].y * inv, a[1].x * inv, a[1].y * inv);
              qv.y = pack_e4m3x4(a[2].x * inv, a[2].y * inv, a[3].x * inv, a[3].y * inv);
              qv.z = pack_e4m3x4(a[4].x * inv, a[4].y * inv, a[5].x * inv, a[5].y * inv);
              qv.w = pack_e4m3x4(a[6].x * inv, a[6].y * inv, a[7].x * inv, a[7].y * inv);
              const int col0 = j * PASS_STRIDE + h * HCB + c * 16;  // column inside the pass's 128
              *reinterpret_cast<uint4*>(irow + sw128(r, col0 / 16)) = qv;
              if (p.dbg_inter != nullptr && fi >= 0 && !dead && ti.e != SHARED_E)
                *reinterpret_cast<uint4*>(p.dbg_inter + static_cast<size_t>(ti.row0 + r) * N_HALF + ti.chunk * CHUNK_COLS + ps * 128 + col0) = qv;
            }
          }
          if (p.dbg_inter_scale != nullptr && fi >= 0 && h == 0 && !dead && ti.e != SHARED_E)
            p.dbg_inter_scale[static_cast<size_t>(ti.row0 + r) * NPT + ti.chunk * NP + ps] = my_scale;
          // publish this pass's 128 intermediate columns to the tensor core (async proxy)
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) { if (PAIR && !leader) mbar_arrive_cluster(at_leader(&S.inter_ready[ps])); else mbar_arrive(&S.inter_ready[ps]); }
          PROF_ADD(pe_silu);
        }

        // ---------------- down projection, routing weight, bf16 partial rows.
        // Every epilogue thread is past the last pass's barrier, so nobody reads this tile's
        // activation scales any more: the next tile's are staged while the down slabs run.
        if (has_next) stage_ids(it + 1);
        for (int hb = 0; hb < NHB; ++hb) {
#pragma unroll
          for (int i = 0; i < TCOLS / 2; ++i) acc[i] = make_float2(0.f, 0.f);
          if (has_next) {
            if (hb == 1) stage_weight_store(it + 1);
            if (hb >= 1 && hb - 1 < AS_PIECES) as_piece_load(hb - 1);
          }
#pragma unroll
          for (int dk = 0; dk < NP; ++dk) {
#pragma unroll
            for (int j = 0; j < NSPLIT; ++j) {
              // output columns hb*256 + j*BC + h*WC ..: one [128,128] weight-scale block
              const float sc = __fmul_rn(wsd_t[(hb * 2 + (j * BC + h * WC) / 128) * NP + dk], iscale[dk]);
              const uint32_t buf = nt % NBUF;
              TRACE_E(0);
              { PROF_T0();
              if (!dead && !mbar_wait(&S.tmem_full[buf], (nt / NBUF) & 1u, wc, kSiteTmemFull)) dead = true;
              PROF_ADD(pe_wait); PROF_HIST(0, 16 + dk, et == 0); }
              TRACE_E(1);
              PROF_T0();
              if (!dead) promote(j, buf, sc, sc);
              PROF_ADD(pe_down);
              TRACE_E(3);
              ++nt;
            }
          }
          PROF_T0();
          // Neighbouring lanes swap half of their 32-byte pieces first, so that in every store instruction
          // lanes 2i and 2i+1 write 64 contiguous bytes of ONE row: 16 lines per instruction instead of 32.
          // (the guard is made warp-uniform: the shuffles below need every lane of the warp)
          if (!__any_sync(0xFFFFFFFFu, dead) && (MONO_ABLATE & 4) == 0) {
            const bool odd = (lane & 1) != 0;
            const int fi_even = __shfl_sync(0xFFFFFFFFu, fi, lane & ~1), fi_odd = __shfl_sync(0xFFFFFFFFu, fi, lane | 1);
            __nv_bfloat16* row_even = p.partial + (static_cast<size_t>(fi_even < 0 ? 0 : fi_even) * NCH + ti.chunk) * H_DIM + hb * 256 + h * WC;
            __nv_bfloat16* row_odd = p.partial + (static_cast<size_t>(fi_odd < 0 ? 0 : fi_odd) * NCH + ti.chunk) * H_DIM + hb * 256 + h * WC;
#pragma unroll
            for (int j = 0; j < NSPLIT; ++j) {
              __nv_bfloat16* dst_even = row_even + j * BC;
              __nv_bfloat16* dst_odd = row_odd + j * BC;
#pragma unroll
              for (int k2 = 0; k2 < WC / 32; ++k2) {   // pieces 2*k2 and 2*k2+1 of this thread's WC columns of buffer j
                uint32_t lo[8], hi[8], mine[8], theirs[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float2 a = __fmul2_rn(acc[j * (WC / 2) + (2 * k2) * 8 + i], rw2);
                  const float2 b = __fmul2_rn(acc[j * (WC / 2) + (2 * k2 + 1) * 8 + i], rw2);
                  lo[i] = cvt_bf16x2_satfinite(a.x, a.y);
                  hi[i] = cvt_bf16x2_satfinite(b.x, b.y);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  // an even lane keeps its piece 2*k2 and gives away 2*k2+1; an odd lane the other way round
                  const uint32_t send = odd ? lo[i] : hi[i];
                  theirs[i] = (MONO_ABLATE & 256) ? send : __shfl_xor_sync(0xFFFFFFFFu, send, 1);
                  mine[i] = odd ? hi[i] : lo[i];
                }
                const int piece = 2 * k2 + (odd ? 1 : 0);
                // row of the even lane: its own piece from the even lane, the received one from the odd lane
                if (fi_even >= 0) st_global_256_stream(dst_even + piece * 16, odd ? theirs : mine);
                if (fi_odd >= 0) st_global_256_stream(dst_odd + piece * 16, odd ? mine : theirs);
              }
            }
          }
          if (has_next && hb >= 1 && hb - 1 < AS_PIECES) as_piece_store(hb - 1);
          PROF_ADD(pe_store);
        }
      }
      if (et == 0) {
        PROF_STORE(8, pe_wait); PROF_STORE(9, pe_up); PROF_STORE(10, pe_silu); PROF_STORE(11, pe_down);
        PROF_STORE(12, pe_store); PROF_STORE(14, pe_bar);
#if defined(MONO_PROFILE) && !defined(MONO_TRACE)
        p.ws->prof[blockIdx.x][13] = static_cast<uint64_t>(clock64() - pe_start);
        for (int i = 0; i < 24; ++i) p.ws->prof[blockIdx.x][16 + i] = S.whist[0][i];
#endif
      }
    }
  }

  // teardown of phase 2: when aborting, give in-flight bulk copies and MMAs time to land
  if (aborted(ws)) __nanosleep(200000);
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();  // nothing of the peer is still signalling this CTA, or reading its tensor memory
  else __syncthreads();
  // Registers go back to the launch split only now, behind the barrier. If the producer warps asked
  // for theirs back right after their own loops (a CTA without tiles reaches that point at once), they
  // could take back what they had just released before the epilogue warps were served, and the
  // epilogue's setmaxnreg.inc would then wait for registers that nobody releases any more.
  if (warp < 4) reg_inc<REGS_LAUNCH>(); else reg_dec<REGS_LAUNCH>();
  if (warp == WARP_MMA) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }

  alive = grid_sync(wc, 2, &S.flag) && alive;
  if (bid == 0 && tid == 0) ws->phase_ns[3] = globaltimer_ns();
  if (!alive) return;

  // ================================================================ phase 3
  // out[t,:] = bf16( sum_k partial[t*8+k,:] * out_scale (+ residual[t,:]) ), k ascending, fp32
  // (kernel/qwen_tp/src/prefill_mono_final_nb.cu:1377-1460). Under expert parallelism slots
  // this rank does not own were never written and are skipped (kernel/qwen_ep/...:1459-1481).
  {
    constexpr int W = 8;                    // bf16 per 16-byte vector
    constexpr int HV = H_DIM / W;
    const size_t out_vec = static_cast<size_t>(T) * HV;
    const int ncomp = tp_on ? (kGrid - p.tp_ncomm) : kGrid;
    const int nchunk = tp_on ? p.tp_nchunk : 1;
    const uint32_t seq = (p.tp_seqctr != nullptr) ? ld_relaxed_gpu(&ws->tp_seq_pub) : p.tp_seq;

    // ---- the all-reduce of the ranks' partial outputs, inside the kernel (only when tp_on)
    // Chunked one-shot all-reduce (kernel/qwen_tp/src/prefill_mono_final_nb.cu:1461-1504): once every rank has
    // summed chunk c, each rank reduces its 1/world share of the chunk across the ranks with multimem.ld_reduce
    // and writes the result back to every rank with multimem.st. A rank's share of a chunk is cut into pieces of
    // PIECE 16-byte vectors that CTAs take from a counter: the `ncomm` communication CTAs from the start, and
    // every summing CTA as soon as it has finished its own sums, so that the tail of the transfer has the whole
    // grid's loads in flight.
    constexpr int UN = 8;                                      // 16-byte reduce-loads in flight per thread
    constexpr size_t PIECE = static_cast<size_t>(UN) * BLOCK;  // vectors per piece (48 KB)
    constexpr size_t ALIGN = 32;                               // shares start on 512-byte boundaries
    const size_t out_mv = static_cast<size_t>(T) * H_DIM / 8;
    auto share_of = [&](int c, size_t& s_lo, size_t& s_hi) {
      const size_t lo = out_mv * c / nchunk, hi = out_mv * (c + 1) / nchunk;
      const size_t ng = (hi - lo + ALIGN - 1) / ALIGN;
      s_lo = lo + (ng * p.tp_rank / p.tp_world) * ALIGN;
      s_hi = lo + (ng * (p.tp_rank + 1) / p.tp_world) * ALIGN;
      s_lo = s_lo < hi ? s_lo : hi;
      s_hi = s_hi < hi ? s_hi : hi;
    };
    auto rank_barrier = [&](int slot) -> bool {
      // arrive on every peer's window, then wait for every peer on mine
      for (int rk = 0; rk < p.tp_world; ++rk)
        st_release_sys(p.tp_pads[rk] + static_cast<size_t>(slot) * p.tp_world + p.tp_rank, seq);
      for (int rk = 0; rk < p.tp_world; ++rk) {
        const uint32_t* w = p.tp_pads[p.tp_rank] + static_cast<size_t>(slot) * p.tp_world + rk;
        const uint64_t t0 = globaltimer_ns();
        uint32_t polls = 0;
        while (ld_acquire_sys(w) < seq) {
          if ((++polls & 15u) == 0u) {
            if (aborted(ws)) return false;
            if (globaltimer_ns() - t0 > p.timeout_ns) {
              report_error(ws, kErrRankBarrier, static_cast<uint32_t>(slot), static_cast<uint32_t>(rk), seq);
              return false;
            }
          }
        }
      }
      return true;
    };
    // the peer's window when the group has two ranks and the caller passed the table of windows
    __nv_bfloat16* const peer_pair = (tp_on && p.tp_peers != nullptr && p.tp_world == 2) ? p.tp_peers[1 - p.tp_rank] : nullptr;
    // Whole CTA: take pieces of this rank's share of chunk c until none is left. False when the launch aborts.
    // Waits that end only when another bounded wait of this launch has ended (a chunk is opened behind a rank
    // barrier; the closer waits for every piece) get twice the limit, so that the status word names the wait
    // that actually ran out, not one queued behind it.
    const WaitCtx wc_dep{p.ws, 2 * p.timeout_ns};
    auto reduce_pieces = [&](int c) -> bool {
      if (tid == 0)
        S.flag = wait_counter_ge(&ws->tp_open[c], 1u, wc_dep, kErrChunkReady, static_cast<uint32_t>(16 + c)) ? 1u : 0u;
      __syncthreads();
      const bool open = S.flag != 0u;
      __syncthreads();
      if (!open) return false;
      size_t s_lo, s_hi;
      share_of(c, s_lo, s_hi);
      const uint32_t npieces = static_cast<uint32_t>((s_hi - s_lo + PIECE - 1) / PIECE);
      uint32_t mine = 0;
      for (;;) {
        if (tid == 0) S.flag = atomicAdd(&ws->tp_piece[c], 1u);
        __syncthreads();
        const uint32_t j = S.flag;
        __syncthreads();
        if (j >= npieces) break;
        const size_t base = s_lo + static_cast<size_t>(j) * PIECE + tid;
        uint32_t x[UN][4];
        bool live[UN];
        if (peer_pair != nullptr) {
          // Two ranks: read the peer's copy over NVLink, add this rank's own copy from local memory, write the
          // sum to both. Per GPU and direction that moves the output once (half read by the peer, half written to
          // it); the multicast form makes the switch fetch this rank's own copy over NVLink as well and deliver
          // the result to both: one and a half times the traffic for the same bits. (From three ranks on the
          // in-switch reduction and multicast store move less than peer loads and stores would.)
          uint32_t y[UN][4];
#pragma unroll
          for (int u = 0; u < UN; ++u) {
            const size_t v = base + static_cast<size_t>(u) * BLOCK;
            live[u] = v < s_hi;
            if (live[u]) {
              ld_relaxed_sys_b128(peer_pair + v * 8, x[u][0], x[u][1], x[u][2], x[u][3]);
              const uint4 own = __ldcg(reinterpret_cast<const uint4*>(p.out + v * 8));
              y[u][0] = own.x; y[u][1] = own.y; y[u][2] = own.z; y[u][3] = own.w;
            }
          }
#pragma unroll
          for (int u = 0; u < UN; ++u) {
            const size_t v = base + static_cast<size_t>(u) * BLOCK;
            if (live[u]) {
              uint4 r;
              r.x = add_bf16x2_f32(x[u][0], y[u][0]); r.y = add_bf16x2_f32(x[u][1], y[u][1]);
              r.z = add_bf16x2_f32(x[u][2], y[u][2]); r.w = add_bf16x2_f32(x[u][3], y[u][3]);
              *reinterpret_cast<uint4*>(p.out + v * 8) = r;
              st_relaxed_sys_b128(peer_pair + v * 8, r.x, r.y, r.z, r.w);
            }
          }
          ++mine;
          continue;
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const size_t v = base + static_cast<size_t>(u) * BLOCK;
          live[u] = v < s_hi;
          if (live[u]) multimem_ld_reduce_bf16x8(p.tp_mc + v * 8, x[u][0], x[u][1], x[u][2], x[u][3]);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const size_t v = base + static_cast<size_t>(u) * BLOCK;
          if (live[u]) multimem_st_b128(p.tp_mc + v * 8, x[u][0], x[u][1], x[u][2], x[u][3]);
        }
        ++mine;
      }
      if (mine > 0) {
        __threadfence_system();   // the stores of these pieces have reached every rank
        __syncthreads();
        if (tid == 0) atomicAdd(&ws->tp_pieces_done, mine);
      }
      return true;
    };

    if (!tp_on || bid < ncomp) {
      const size_t stride = static_cast<size_t>(ncomp) * BLOCK;
      for (int c = 0; c < nchunk; ++c) {
        const size_t c_lo = out_vec * c / nchunk, c_hi = out_vec * (c + 1) / nchunk;
        for (size_t iv = c_lo + static_cast<size_t>(bid) * BLOCK + tid; iv < c_hi; iv += stride) {
          const size_t tok = iv / HV;
          const int hv = static_cast<int>(iv % HV);
          int own[TOP_K];
          if constexpr (EP_BUILD) {
            const int4* o = reinterpret_cast<const int4*>(p.topk_ids + tok * TOP_K);
            const int4 o0 = o[0], o1 = o[1];
            own[0] = o0.x; own[1] = o0.y; own[2] = o0.z; own[3] = o0.w;
            own[4] = o1.x; own[5] = o1.y; own[6] = o1.z; own[7] = o1.w;
          }
          float s[W];
#pragma unroll
          for (int i = 0; i < W; ++i) s[i] = 0.f;
          // partial rows of the token: slot-major, chunk-minor, summed in that order
          uint4 raw[TOP_K * NCH];
#pragma unroll
          for (int k = 0; k < TOP_K * NCH; ++k) {
            bool mine = true;
            if constexpr (EP_BUILD) mine = own[k / NCH] >= 0;
            raw[k] = make_uint4(0u, 0u, 0u, 0u);
            if (mine)
              raw[k] = __ldcg(reinterpret_cast<const uint4*>(p.partial + (tok * (TOP_K * NCH) + k) * H_DIM + hv * W));
          }
#pragma unroll
          for (int k = 0; k < TOP_K * NCH; ++k) {
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&raw[k]);
#pragma unroll
            for (int i = 0; i < W; ++i) s[i] += __bfloat162float(b[i]);
          }
          __nv_bfloat16 o[W];
          if (p.sh_on) {
            // out = bf16(routed * out_scale + (shared expert's rows, already times its gate) + residual)
            float base[W];
#pragma unroll
            for (int i = 0; i < W; ++i) base[i] = 0.f;
            if (static_cast<int>(tok / TILE_M) % p.sh_parts == p.sh_part) {   // rows this launch computed
#pragma unroll
              for (int c = 0; c < NCH; ++c) {
                const uint4 sr = __ldcg(reinterpret_cast<const uint4*>(
                    p.partial + ((static_cast<size_t>(numel) + tok) * NCH + c) * H_DIM + hv * W));
                const __nv_bfloat16* sb = reinterpret_cast<const __nv_bfloat16*>(&sr);
#pragma unroll
                for (int i = 0; i < W; ++i) base[i] += __bfloat162float(sb[i]);
              }
            }
            if (p.residual != nullptr) {
              const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + iv * W);
              const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(&rr);
#pragma unroll
              for (int i = 0; i < W; ++i) base[i] += __bfloat162float(rb[i]);
            }
#pragma unroll
            for (int i = 0; i < W; ++i) o[i] = __float2bfloat16(__fmaf_rn(s[i], p.out_scale, base[i]));
          } else if (p.residual != nullptr) {
            const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + iv * W);
            const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(&rr);
#pragma unroll
            for (int i = 0; i < W; ++i) o[i] = __float2bfloat16(__fmaf_rn(s[i], p.out_scale, __bfloat162float(rb[i])));
          } else {
#pragma unroll
            for (int i = 0; i < W; ++i) o[i] = __float2bfloat16(__fmul_rn(s[i], p.out_scale));
          }
          *reinterpret_cast<uint4*>(p.out + iv * W) = *reinterpret_cast<const uint4*>(o);
        }
        if (!tp_on) continue;
        __threadfence_system();  // a peer's communication block reads these bytes through the multicast alias
        __syncthreads();
        if (tid == 0) atomicAdd(&ws->tp_ready[c], 1u);
      }
      if (tp_on) {   // sums done: join the transfer of whatever is not reduced yet
        for (int c = 0; c < nchunk; ++c)
          if (!reduce_pieces(c)) break;
      }
    } else {
      // ---------------------------------------------------------- communication blocks
      // Block cb opens the chunks c = cb, cb + ncomm, ...: it waits until this rank's summing blocks have
      // finished the chunk, meets the peers' block cb at a rank barrier (window slot c) and raises tp_open[c].
      // With ncomm >= nchunk (the usual shapes) every chunk has its own opener, so a chunk opens as soon as the
      // slowest rank has summed it. Then it takes pieces like everybody else.
      const int cb = bid - ncomp;
      bool ok = true;
      for (int c = cb; c < nchunk && ok; c += p.tp_ncomm) {
        if (tid == 0) {
          ok = wait_counter_ge(&ws->tp_ready[c], static_cast<uint32_t>(ncomp), wc, kErrChunkReady, static_cast<uint32_t>(c));
          if (ok) ok = rank_barrier(c);
          if (ok) {
            __threadfence();
            atomicExch(&ws->tp_open[c], 1u);
          }
          S.flag = ok ? 1u : 0u;
        }
        __syncthreads();
        ok = S.flag != 0u;
        __syncthreads();
      }
      for (int c = 0; c < nchunk && ok; ++c) ok = reduce_pieces(c);
      // Block 0 closes the launch: when every piece of this rank's shares is out, it meets the peers at the last
      // rank barrier. Behind it every rank's stores into this rank's buffer have landed; the kernel cannot
      // complete before this block returns.
      if (cb == 0 && tid == 0 && ok) {
        uint32_t total = 0;
        for (int c = 0; c < nchunk; ++c) {
          size_t s_lo, s_hi;
          share_of(c, s_lo, s_hi);
          total += static_cast<uint32_t>((s_hi - s_lo + PIECE - 1) / PIECE);
        }
        if (wait_counter_ge(&ws->tp_pieces_done, total, wc_dep, kErrDoneFlag, 0) && rank_barrier(nchunk * p.tp_ncomm)) {
          __threadfence();
          atomicExch(&ws->tp_done_flag, 1u);
        }
      }
      __syncthreads();
    }
  }
  if (bid == 0 && tid == 0) ws->phase_ns[4] = globaltimer_ns();
}

// ------------------------------------------------------------------ host side
uint64_t g_timeout_ns = 2000000000ull;  // bound of every device-side wait: 2 s
float* g_dbg_acc = nullptr;
uint8_t* g_dbg_inter = nullptr;
float* g_dbg_inter_scale = nullptr;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is fetched through the runtime, so the library has no link-time
// dependency on libcuda and its accessors load on a machine without a driver.
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D u8 tensor [rows, cols] row-major, box box_rows x 128 bytes, 128-byte swizzle.
int make_u8_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t gd[2] = {cols, rows};
  cuuint64_t gs[1] = {cols};
  cuuint32_t bx[2] = {128u, box_rows};
  cuuint32_t es[2] = {1u, 1u};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gd, gs, bx, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// 2-D bf16 tensor [rows, cols] row-major, box box_rows x 64 elements (128 bytes), 128-byte swizzle;
// rows past the end read as zero.
int make_bf16_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t gd[2] = {cols, rows};
  cuuint64_t gs[1] = {cols * 2};
  cuuint32_t bx[2] = {64u, box_rows};
  cuuint32_t es[2] = {1u, 1u};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gd, gs, bx, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// Plan / run split. What a launch needs besides its arguments depends only on the device (the kernel's
// shared-memory attribute) and on the weight tensors (their TMA descriptors: base address + the compiled
// extents). Both are made once and kept: a descriptor per (kind, base address, rows) in a small table, the
// attribute once per device. The reference re-encodes both descriptors and re-sets the attribute on every
// call (kernel/qwen_tp/src/prefill_mono_final_nb.cu:1611-1639, :1655).
struct MapKey {
  const void* base;
  uint64_t rows;
  int kind;  // 0 up weights, 1 down weights, 2 activations (router), 3 router weight
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && kind == o.kind; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (std::hash<uint64_t>()(k.rows) * 1000003u) ^ static_cast<size_t>(k.kind) << 1;
  }
};
std::mutex g_plan_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
unsigned long long g_map_hits = 0, g_map_misses = 0;
constexpr size_t kMaxCachedMaps = 4096;   // far more than the MoE layers of a model; beyond it the table restarts
bool g_attr_set[64] = {};

// Copies the cached descriptor into *dst, encoding it first if this tensor has not been seen.
int cached_map(CUtensorMap* dst, int kind, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  const MapKey key{base, rows, kind};
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    ++g_map_hits;
    *dst = it->second;
    return 0;
  }
  ++g_map_misses;
  CUtensorMap m;
  const int rc = (kind <= 1) ? make_u8_map(&m, base, rows, cols, box_rows) : make_bf16_map(&m, base, rows, cols, box_rows);
  if (rc != 0) return rc;
  if (g_maps.size() >= kMaxCachedMaps) g_maps.clear();
  g_maps.emplace(key, m);
  *dst = m;
  return 0;
}

cudaError_t ensure_kernel_attribute(int dev) {
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  if (dev >= 0 && dev < 64 && g_attr_set[dev]) return cudaSuccess;
  const cudaError_t err = cudaFuncSetAttribute(moe_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_SMEM);
  if (err == cudaSuccess && dev >= 0 && dev < 64) g_attr_set[dev] = true;
  return err;
}

}  // namespace
}  // namespace mono

using namespace mono;

extern "C" {

size_t prefill_wgmma_workspace_bytes() { return sizeof(Workspace); }
int prefill_wgmma_num_experts() { return E; }
int prefill_wgmma_num_experts_local() { return E_LOCAL; }
int prefill_wgmma_ep_capable() { return EP_BUILD ? 1 : 0; }
int prefill_wgmma_top_k() { return TOP_K; }
int prefill_wgmma_max_tiles() { return MAX_TILES; }
int prefill_wgmma_grid_size() { return kGrid; }
int prefill_wgmma_k_dim() { return K_DIM; }
int prefill_wgmma_h_dim() { return H_DIM; }
int prefill_wgmma_fused_renorm() { return 1; }
int prefill_wgmma_router_mode() { return ROUTER_MODE; }
int prefill_wgmma_n_group() { return N_GROUP; }
int prefill_wgmma_topk_group() { return TOPK_GROUP; }
int prefill_wgmma_n_up() { return N_UP; }
int prefill_wgmma_n_half() { return N_HALF; }
int prefill_wgmma_block_m() { return TILE_M; }
int prefill_wgmma_tp_max_c() { return kTpMaxChunks; }
int prefill_wgmma_tp_align() { return 32; }
int prefill_wgmma_tp_mm() { return 8; }
int prefill_wgmma_tp_has_devseq() { return 1; }
int prefill_wgmma_tp_seq_bytes() { return static_cast<int>(sizeof(uint32_t)); }
int prefill_wgmma_tp_has_residual() { return 1; }
int prefill_wgmma_tp_pad_words(int nchunk, int ncomm, int world) { return (nchunk * ncomm + 1) * world; }
int prefill_wgmma_up_pipe() { return SB; }
int prefill_wgmma_dn_pipe() { return SB; }
int prefill_wgmma_a_stages() { return SA; }
int prefill_wgmma_shm_total() { return DYN_SMEM + static_cast<int>(sizeof(SharedState)); }

// ---- additions of this build (new capability = new symbol)
int prefill_wgmma_arch() { return 100; }
// 1: tiles run as pairs on clusters of two CTAs; the total_tiles word of the workspace then counts pairs
int prefill_wgmma_cta_pair() { return PAIR ? 1 : 0; }
// Chunks the intermediate is processed in (1 unless wider than 512 columns). output_accum must hold
// num_tokens * top_k * chunks rows of H bf16 values: with 1 or 2 chunks the reference's fp32 [T*8, H]
// allocation is large enough, beyond that the caller sizes it from this accessor.
int prefill_wgmma_partial_chunks() { return NCH; }
int prefill_wgmma_block_threads() { return BLOCK; }
int prefill_wgmma_stable_sort() { return 1; }
// Byte offset of the 32-bit status word inside the workspace and the bytes that follow it
// (status, abort flag, two detail words). 0 after a successful launch.
int prefill_wgmma_status_offset() { return static_cast<int>(offsetof(Workspace, status)); }
int prefill_wgmma_status_bytes() { return 16; }
int prefill_wgmma_counts_offset() { return static_cast<int>(offsetof(Workspace, expert_counts)); }
int prefill_wgmma_offsets_offset() { return static_cast<int>(offsetof(Workspace, expert_offsets)); }
int prefill_wgmma_total_tiles_offset() { return static_cast<int>(offsetof(Workspace, total_tiles)); }
int prefill_wgmma_phase_ns_offset() { return static_cast<int>(offsetof(Workspace, phase_ns)); }
int prefill_wgmma_prof_offset() { return static_cast<int>(offsetof(Workspace, prof)); }
// Upper bound, in microseconds, of every device-side wait of later launches.
void prefill_wgmma_set_wait_timeout_us(unsigned long long us) { g_timeout_ns = us * 1000ull; }
// Debug dump targets for later launches (device pointers, or null to switch off):
// acc [T*8, N_UP] fp32 raw gate|up sums, inter [T*8, N_HALF] e4m3, inter_scale [T*8, N_HALF/128] fp32,
// all indexed by sorted row.
void prefill_wgmma_set_debug(void* acc, void* inter, void* inter_scale) {
  g_dbg_acc = static_cast<float*>(acc);
  g_dbg_inter = static_cast<uint8_t*>(inter);
  g_dbg_inter_scale = static_cast<float*>(inter_scale);
}

// Plan step, optional: make (or find) the descriptors of a layer's weights and set the kernel's attribute on
// the current device now, so that the first launch of that layer does not pay for it. Launches look the
// descriptors up by the weights' addresses; a layer that was never prepared is prepared by its first launch.
// Returns 0, -2 / -3 (descriptor encoding failed) or a cudaError_t.
int prefill_wgmma_plan_prepare(const uint8_t* up_w_fp8, const uint8_t* down_w_fp8) {
  if (up_w_fp8 == nullptr || down_w_fp8 == nullptr) return -104;
  CUtensorMap tmp;
  if (cached_map(&tmp, 0, up_w_fp8, static_cast<uint64_t>(E_LOCAL) * N_UP, K_DIM, HCB) != 0) return -2;
  if (cached_map(&tmp, 1, down_w_fp8, static_cast<uint64_t>(E_LOCAL) * H_DIM, N_HALF, HCB) != 0) return -3;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err == cudaSuccess) err = ensure_kernel_attribute(dev);
  return static_cast<int>(err);
}
// Descriptor look-ups served from the table / encoded anew since the library was loaded.
void prefill_wgmma_plan_stats(unsigned long long* hits, unsigned long long* misses) {
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  if (hits != nullptr) *hits = g_map_hits;
  if (misses != nullptr) *misses = g_map_misses;
}
// Forget every cached descriptor (weights were freed and their addresses will be reused for other shapes).
void prefill_wgmma_plan_reset() {
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  g_maps.clear();
}

// The shared expert of a launch (all null / zero: none).
struct SharedExpertArgs {
  const uint8_t* up_w_fp8;      // e4m3 [2 * N_HALF, K], gate rows then up rows
  const float* up_w_scales;     // fp32 [2 * N_HALF / 128, K / 128]
  const uint8_t* down_w_fp8;    // e4m3 [H, N_HALF]
  const float* down_w_scales;   // fp32 [H / 128, N_HALF / 128]
  const void* gate_bf16;        // bf16 [K] or null
  float* gate_scratch;          // fp32 [T], required with gate_bf16
  int part, parts;
};

// Common launcher. router_w == nullptr: `logits` holds the caller's router logits. Otherwise
// router_w is the bf16 router weight [E, K] and `logits` is the [T, E] fp32 buffer the kernel fills.
static int launch_common(const void* router_w, float* logits_buf, const float* logits, int num_tokens, int block_m,
                         void* workspace,
                                    size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                    float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                    const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                    int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                    void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                    int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                    void* tp_seqctr, const void* tp_residual, float out_scale,
                                    const int32_t* expert_map, cudaStream_t stream,
                                    const SharedExpertArgs* sh = nullptr, void* tp_peers = nullptr) {
  (void)block_m;  // the tile height is the compiled TILE_M
  if (router_w != nullptr && PAIR) return -106;  // the pair build has no router linear
  if (sh != nullptr && PAIR) return -108;        // nor the shared expert
  if (router_w != nullptr) logits = logits_buf;
  // order of the checks as in kernel/qwen_ep/src/prefill_mono_final_nb.cu:1650-1660
  if (workspace == nullptr || workspace_bytes < sizeof(Workspace)) return -100;
  if (EP_BUILD && expert_map == nullptr) return -120;
  if (!EP_BUILD && expert_map != nullptr) return -121;
  if (num_tokens <= 0) return -101;
  const long long numel = static_cast<long long>(num_tokens) * TOP_K;
  const long long sh_tiles = (sh != nullptr) ? (num_tokens + TILE_M - 1) / TILE_M : 0;
  if ((numel / TILE_M + E_LOCAL + sh_tiles) * NCH > MAX_TILES) return -102;
  if (logits == nullptr || act_bf16 == nullptr || act_fp8 == nullptr || act_scales == nullptr ||
      up_w_fp8 == nullptr || up_w_scales == nullptr || down_w_fp8 == nullptr || down_w_scales == nullptr ||
      output_accum == nullptr || topk_ids == nullptr || topk_weights == nullptr || sorted_token_ids == nullptr ||
      bf16_output == nullptr)
    return -104;
  if (sh != nullptr) {
    if (sh->up_w_fp8 == nullptr || sh->up_w_scales == nullptr || sh->down_w_fp8 == nullptr ||
        sh->down_w_scales == nullptr || (sh->gate_bf16 != nullptr && sh->gate_scratch == nullptr))
      return -109;
    if (sh->parts < 1 || sh->part < 0 || sh->part >= sh->parts) return -109;
  }
  if (tp_mc != nullptr && tp_ncomm > 0) {
    if (tp_nchunk < 1 || tp_nchunk > kTpMaxChunks) return -110;
    if (tp_ncomm >= kGrid) return -111;
    if (tp_world < 1 || tp_rank < 0 || tp_rank >= tp_world) return -112;
    if (tp_pads == nullptr) return -113;
    if ((static_cast<size_t>(num_tokens) * H_DIM) % (8 * static_cast<size_t>(tp_nchunk))) return -114;
  }

  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return static_cast<int>(err);
  int sm_count = 0;
  err = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (sm_count < kGrid) return -103;

  Params p{};
  p.logits = logits;
  p.num_tokens = num_tokens;
  p.ws = static_cast<Workspace*>(workspace);
  p.topk_ids = topk_ids;
  p.topk_weights = topk_weights;
  p.sorted_ids = sorted_token_ids;
  p.act_bf16 = static_cast<const __nv_bfloat16*>(act_bf16);
  p.act_fp8 = act_fp8;
  p.act_scales = act_scales;
  p.up_w_scales = up_w_scales;
  p.down_w_scales = down_w_scales;
  p.partial = reinterpret_cast<__nv_bfloat16*>(output_accum);
  p.out = static_cast<__nv_bfloat16*>(bf16_output);
  p.router_bias = router_bias;
  p.expert_map = expert_map;
  p.tp_mc = static_cast<__nv_bfloat16*>(tp_mc);
  p.tp_pads = static_cast<uint32_t**>(tp_pads);
  p.tp_rank = tp_rank;
  p.tp_world = tp_world;
  p.tp_nchunk = tp_nchunk;
  p.tp_ncomm = tp_ncomm;
  p.tp_seq = tp_seq;
  p.tp_seqctr = static_cast<uint32_t*>(tp_seqctr);
  p.tp_peers = static_cast<__nv_bfloat16**>(tp_peers);
  p.residual = static_cast<const __nv_bfloat16*>(tp_residual);
  p.out_scale = out_scale;
  p.timeout_ns = g_timeout_ns;
  p.dbg_acc = g_dbg_acc;
  p.dbg_inter = g_dbg_inter;
  p.dbg_inter_scale = g_dbg_inter_scale;

  int rc = cached_map(&p.tm_up, 0, up_w_fp8, static_cast<uint64_t>(E_LOCAL) * N_UP, K_DIM, HCB);
  if (rc != 0) {
    fprintf(stderr, "up-projection tensor map failed: %d\n", rc);
    return -2;
  }
  rc = cached_map(&p.tm_down, 1, down_w_fp8, static_cast<uint64_t>(E_LOCAL) * H_DIM, N_HALF, HCB);
  if (rc != 0) {
    fprintf(stderr, "down-projection tensor map failed: %d\n", rc);
    return -3;
  }
  if (sh != nullptr) {
    p.sh_on = 1;
    p.sh_up_scales = sh->up_w_scales;
    p.sh_down_scales = sh->down_w_scales;
    p.sh_gate = static_cast<const __nv_bfloat16*>(sh->gate_bf16);
    p.sh_gate_w = sh->gate_scratch;
    p.sh_part = sh->part;
    p.sh_parts = sh->parts;
    rc = cached_map(&p.tm_sh_up, 0, sh->up_w_fp8, static_cast<uint64_t>(N_UP), K_DIM, HCB);
    if (rc == 0) rc = cached_map(&p.tm_sh_down, 1, sh->down_w_fp8, static_cast<uint64_t>(H_DIM), N_HALF, HCB);
    if (rc != 0) {
      fprintf(stderr, "shared-expert tensor map failed: %d\n", rc);
      return -5;
    }
  } else {
    p.sh_parts = 1;
  }
  if (router_w != nullptr) {
    p.logits_out = logits_buf;
    rc = cached_map(&p.tm_x, 2, act_bf16, static_cast<uint64_t>(num_tokens), K_DIM, TILE_M);
    if (rc == 0) rc = cached_map(&p.tm_rw, 3, router_w, E, K_DIM, E);
    if (rc != 0) {
      fprintf(stderr, "router tensor map failed: %d\n", rc);
      return -4;
    }
  }

  err = ensure_kernel_attribute(dev);
  if (err != cudaSuccess) return static_cast<int>(err);
  // only the head of the workspace has to start at zero (barrier counters, status, chunk counters)
  err = cudaMemsetAsync(workspace, 0, kWorkspaceZeroBytes, stream);
  if (err != cudaSuccess) return static_cast<int>(err);

  if constexpr (PAIR) {
    // 74 clusters of two CTAs; both CTAs of a cluster run on the two SMs of one TPC
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kGrid);
    cfg.blockDim = dim3(BLOCK);
    cfg.dynamicSmemBytes = DYN_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    static int clusters_fit = -1;   // every cluster has to be resident at once (grid barriers)
    if (clusters_fit < 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, moe_prefill_kernel, &cfg) != cudaSuccess) n = 0;
      clusters_fit = n;
    }
    if (clusters_fit < kGrid / 2) {
      fprintf(stderr, "only %d of %d two-CTA clusters can be resident\n", clusters_fit, kGrid / 2);
      return -107;
    }
    err = cudaLaunchKernelEx(&cfg, moe_prefill_kernel, p);
    if (err != cudaSuccess) {
      fprintf(stderr, "kernel launch failed: %s\n", cudaGetErrorString(err));
      return static_cast<int>(err);
    }
    return 0;
  }
  moe_prefill_kernel<<<kGrid, BLOCK, DYN_SMEM, stream>>>(p);
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    fprintf(stderr, "kernel launch failed: %s\n", cudaGetErrorString(err));
    return static_cast<int>(err);
  }
  return 0;
}

int launch_prefill_moe_wgmma_q1_ep2(const float* logits, int num_tokens, int block_m, void* workspace,
                                    size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                    float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                    const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                    int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                    void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                    int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                    void* tp_seqctr, const void* tp_residual, float out_scale,
                                    const int32_t* expert_map, cudaStream_t stream) {
  return launch_common(nullptr, nullptr, logits, num_tokens, block_m, workspace, workspace_bytes, act_bf16, act_fp8,
                       act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales, output_accum, topk_ids,
                       topk_weights, sorted_token_ids, bf16_output, router_bias, tp_mc, tp_pads, tp_rank, tp_world,
                       tp_nchunk, tp_ncomm, tp_seq, tp_seqctr, tp_residual, out_scale, expert_map, stream);
}

// The _ep2 entry plus tp_peers: a device array of tp_world pointers, every rank's address of the output window
// (bf16_output on that rank). With two ranks the in-kernel reduce then reads the peer's copy directly instead
// of going through the multicast alias (two thirds of the NVLink traffic, the same bits); with more ranks, or a null
// table, it is the multicast reduce of the _ep2 entry.
int prefill_wgmma_tp_has_peer_reduce() { return 1; }
int launch_prefill_moe_wgmma_q1_ep3(const float* logits, int num_tokens, int block_m, void* workspace,
                                    size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                    float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                    const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                    int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                    void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                    int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                    void* tp_seqctr, const void* tp_residual, float out_scale,
                                    const int32_t* expert_map, void* tp_peers, cudaStream_t stream) {
  return launch_common(nullptr, nullptr, logits, num_tokens, block_m, workspace, workspace_bytes, act_bf16, act_fp8,
                       act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales, output_accum, topk_ids,
                       topk_weights, sorted_token_ids, bf16_output, router_bias, tp_mc, tp_pads, tp_rank, tp_world,
                       tp_nchunk, tp_ncomm, tp_seq, tp_seqctr, tp_residual, out_scale, expert_map, stream, nullptr,
                       tp_peers);
}

// The router linear inside the launch: router_w_bf16 is the gate weight [E, K] in bf16 (the checkpoints
// of both model families store it so) and logits_out a [T, E] fp32 buffer that receives the logits the
// kernel routed on. Everything from num_tokens on is the argument list of the _ep2 entry.
// -105: router_w_bf16 or logits_out is null.
int prefill_wgmma_has_router_gemv() { return PAIR ? 0 : 1; }
int launch_prefill_moe_wgmma_q1_gemv(const void* router_w_bf16, float* logits_out, int num_tokens, int block_m,
                                     void* workspace, size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                     float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                     const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                     int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                     void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                     int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                     void* tp_seqctr, const void* tp_residual, float out_scale,
                                     const int32_t* expert_map, cudaStream_t stream) {
  if (router_w_bf16 == nullptr || logits_out == nullptr) return -105;
  return launch_common(router_w_bf16, logits_out, nullptr, num_tokens, block_m, workspace, workspace_bytes, act_bf16,
                       act_fp8, act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales, output_accum, topk_ids,
                       topk_weights, sorted_token_ids, bf16_output, router_bias, tp_mc, tp_pads, tp_rank, tp_world,
                       tp_nchunk, tp_ncomm, tp_seq, tp_seqctr, tp_residual, out_scale, expert_map, stream);
}

// The gated shared expert inside the same launch. The argument list of the _ep2 entry, then the shared
// expert: block-FP8 weights in the layout of one routed expert ([2 * N_HALF, K] and [H, N_HALF] with their
// [128,128] scales), an optional bf16 gate vector [K] (the row is multiplied by sigmoid(x . g); null: by 1) with
// its [T] fp32 scratch, and (sh_part, sh_parts): this launch computes the shared expert for the 128-token tiles
// j with j % sh_parts == sh_part (expert-parallel ranks split the tokens; 0, 1 otherwise). output_accum has to
// hold num_tokens * (top_k + 1) * partial_chunks rows. out = bf16(out_scale * routed + shared + residual).
// -108: not in the two-CTA build; -109: a shared-expert argument is missing or inconsistent; -5: descriptor.
int prefill_wgmma_has_shared_expert() { return PAIR ? 0 : 1; }
int launch_prefill_moe_wgmma_q1_shared(const float* logits, int num_tokens, int block_m, void* workspace,
                                       size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                       float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                       const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                       int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                       void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                       int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                       void* tp_seqctr, const void* tp_residual, float out_scale,
                                       const int32_t* expert_map, const uint8_t* sh_up_w_fp8,
                                       const float* sh_up_w_scales, const uint8_t* sh_down_w_fp8,
                                       const float* sh_down_w_scales, const void* sh_gate_bf16, float* sh_gate_scratch,
                                       int sh_part, int sh_parts, cudaStream_t stream) {
  const SharedExpertArgs sh{sh_up_w_fp8, sh_up_w_scales, sh_down_w_fp8, sh_down_w_scales, sh_gate_bf16,
                            sh_gate_scratch, sh_part, sh_parts};
  return launch_common(nullptr, nullptr, logits, num_tokens, block_m, workspace, workspace_bytes, act_bf16, act_fp8,
                       act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales, output_accum, topk_ids,
                       topk_weights, sorted_token_ids, bf16_output, router_bias, tp_mc, tp_pads, tp_rank, tp_world,
                       tp_nchunk, tp_ncomm, tp_seq, tp_seqctr, tp_residual, out_scale, expert_map, stream, &sh);
}

int launch_prefill_moe_wgmma_q1_tp2(const float* logits, int num_tokens, int block_m, void* workspace,
                                    size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                    float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                    const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                    int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                    void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                    int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                    void* tp_seqctr, const void* tp_residual, float out_scale,
                                    cudaStream_t stream) {
  return launch_prefill_moe_wgmma_q1_ep2(logits, num_tokens, block_m, workspace, workspace_bytes, act_bf16, act_fp8,
                                         act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales, output_accum,
                                         topk_ids, topk_weights, sorted_token_ids, bf16_output, router_bias, tp_mc,
                                         tp_pads, tp_rank, tp_world, tp_nchunk, tp_ncomm, tp_seq, tp_seqctr,
                                         tp_residual, out_scale, nullptr, stream);
}

int launch_prefill_moe_wgmma_q1_tp(const float* logits, int num_tokens, int block_m, void* workspace,
                                   size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8, float* act_scales,
                                   const uint8_t* up_w_fp8, const float* up_w_scales, const uint8_t* down_w_fp8,
                                   const float* down_w_scales, float* output_accum, int32_t* topk_ids,
                                   float* topk_weights, int32_t* sorted_token_ids, void* bf16_output,
                                   const float* router_bias, void* tp_mc, void* tp_pads, int tp_rank, int tp_world,
                                   int tp_nchunk, int tp_ncomm, uint32_t tp_seq, void* tp_seqctr,
                                   cudaStream_t stream) {
  return launch_prefill_moe_wgmma_q1_tp2(logits, num_tokens, block_m, workspace, workspace_bytes, act_bf16, act_fp8,
                                         act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales, output_accum,
                                         topk_ids, topk_weights, sorted_token_ids, bf16_output, router_bias, tp_mc,
                                         tp_pads, tp_rank, tp_world, tp_nchunk, tp_ncomm, tp_seq, tp_seqctr, nullptr,
                                         1.0f, stream);
}

int launch_prefill_moe_wgmma_q1_router(const float* logits, int num_tokens, int block_m, void* workspace,
                                       size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                       float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                       const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                       int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                       void* bf16_output, const float* router_bias, cudaStream_t stream) {
  return launch_prefill_moe_wgmma_q1_tp(logits, num_tokens, block_m, workspace, workspace_bytes, act_bf16, act_fp8,
                                        act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales, output_accum,
                                        topk_ids, topk_weights, sorted_token_ids, bf16_output, router_bias, nullptr,
                                        nullptr, 0, 1, 1, 0, 0u, nullptr, stream);
}

int launch_prefill_moe_wgmma_q1(const float* logits, int num_tokens, int block_m, void* workspace,
                                size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8, float* act_scales,
                                const uint8_t* up_w_fp8, const float* up_w_scales, const uint8_t* down_w_fp8,
                                const float* down_w_scales, float* output_accum, int32_t* topk_ids,
                                float* topk_weights, int32_t* sorted_token_ids, void* bf16_output,
                                cudaStream_t stream) {
  return launch_prefill_moe_wgmma_q1_router(logits, num_tokens, block_m, workspace, workspace_bytes, act_bf16,
                                            act_fp8, act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales,
                                            output_accum, topk_ids, topk_weights, sorted_token_ids, bf16_output,
                                            nullptr, stream);
}

int launch_prefill_moe_wgmma_q1_ep(const float* logits, int num_tokens, int block_m, void* workspace,
                                   size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8, float* act_scales,
                                   const uint8_t* up_w_fp8, const float* up_w_scales, const uint8_t* down_w_fp8,
                                   const float* down_w_scales, float* output_accum, int32_t* topk_ids,
                                   float* topk_weights, int32_t* sorted_token_ids, void* bf16_output,
                                   const float* router_bias, const int32_t* expert_map, cudaStream_t stream) {
  return launch_prefill_moe_wgmma_q1_ep2(logits, num_tokens, block_m, workspace, workspace_bytes, act_bf16, act_fp8,
                                         act_scales, up_w_fp8, up_w_scales, down_w_fp8, down_w_scales, output_accum,
                                         topk_ids, topk_weights, sorted_token_ids, bf16_output, router_bias, nullptr,
                                         nullptr, 0, 1, 1, 0, 0u, nullptr, nullptr, 1.0f, expert_map, stream);
}


// ---------------------------------------------------------------------------------------------
// Launch without any allocation by the caller or by this library.
//
// Some hosts of this kernel cannot obtain device memory at call time: a serving engine that has
// already handed every free byte of HBM to its KV-cache pool (a late cudaMalloc there fails, or
// evicts what the engine reserved), and latency-sensitive callers for which the implicit
// device-wide synchronisation of cudaMalloc / cudaFree stalls every other stream. For them the
// scratch the kernel needs (workspace, e4m3 activations and their scales, routing results, the
// sort permutation and the bf16 partial rows) lives in the fixed array below, which every GPU
// that loads this library holds from load until the process exits. The caller passes only the
// inputs and the output. The price is a cap on the batch: kNoAllocMaxTokens tokens.
//
// * All calls on one device share the array. It keeps the previous call's contents; the launch
//   clears the part that must start at zero (the workspace). Two calls whose kernels overlap on
//   the GPU (different streams, no ordering between them) race on it: serialise them.
// * The first call on each device resolves the array's device address with cudaGetSymbolAddress
//   (with that device current) and caches it; make that first call outside any stream capture.
constexpr int kNoAllocMaxTokens = (H_DIM <= 2048) ? 256 : (NCH > 1 ? 32 : 64);
constexpr size_t na_align(size_t x) { return (x + 255) / 256 * 256; }
constexpr size_t kNaWorkspace = 0;
constexpr size_t kNaActFp8 = kNaWorkspace + na_align(sizeof(Workspace));
constexpr size_t kNaActScales = kNaActFp8 + na_align(static_cast<size_t>(kNoAllocMaxTokens) * K_DIM);
constexpr size_t kNaTopkIds = kNaActScales + na_align(static_cast<size_t>(kNoAllocMaxTokens) * NK * 4);
constexpr size_t kNaTopkW = kNaTopkIds + na_align(static_cast<size_t>(kNoAllocMaxTokens) * TOP_K * 4);
constexpr size_t kNaSorted = kNaTopkW + na_align(static_cast<size_t>(kNoAllocMaxTokens) * TOP_K * 4);
constexpr size_t kNaPartial = kNaSorted + na_align(static_cast<size_t>(kNoAllocMaxTokens) * TOP_K * 4);
constexpr size_t kNaBytes = kNaPartial + na_align(static_cast<size_t>(kNoAllocMaxTokens) * TOP_K * NCH * H_DIM * 2);

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaBytes];

// Device address of the array on the current device; resolved on first use when `resolve` is set.
static int noalloc_base(unsigned char** out, bool resolve) {
  constexpr int kMaxDevices = 64;
  static unsigned char* base_of_device[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  const cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (dev < 0 || dev >= kMaxDevices) return -131;
  std::lock_guard<std::mutex> lock(mu);
  if (base_of_device[dev] == nullptr && resolve) {
    // In host code the array's name is only a handle: the device address has to be asked for, once per
    // device, with that device current.
    void* ptr = nullptr;
    const cudaError_t e2 = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e2 != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "launch_prefill_moe_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e2));
      return -131;
    }
    base_of_device[dev] = static_cast<unsigned char*>(ptr);
  }
  if (base_of_device[dev] == nullptr) return -131;
  *out = base_of_device[dev];
  return 0;
}

int prefill_wgmma_noalloc_max_tokens() { return kNoAllocMaxTokens; }
// The status words (status, abort flag, two detail words) of the last launch_prefill_moe_noalloc on the
// current device, copied to out[0..3] on `stream`: the workspace of that entry is inside the library, so this
// is how its caller learns of a bounded wait that gave up. out[0] == 0 means success. Enqueue it behind the
// launch on the same stream and read `out` after synchronising (pinned memory makes the copy asynchronous).
// -131 before the first launch on this device; otherwise 0 or a cudaError_t.
int prefill_wgmma_noalloc_status(uint32_t* out, cudaStream_t stream) {
  if (out == nullptr) return -104;
  unsigned char* b = nullptr;
  const int rc = noalloc_base(&b, false);
  if (rc != 0) return rc;
  return static_cast<int>(cudaMemcpyAsync(out, b + kNaWorkspace + offsetof(Workspace, status), 16,
                                          cudaMemcpyDeviceToHost, stream));
}
size_t prefill_wgmma_noalloc_scratch_bytes() { return kNaBytes; }

// Returns 0 on success; -130 when num_tokens exceeds prefill_wgmma_noalloc_max_tokens(); -131 when the
// device address of the scratch array cannot be resolved; otherwise the codes of the other entry points.
int launch_prefill_moe_noalloc(const float* logits, int num_tokens, const void* act_bf16, const uint8_t* up_w_fp8,
                               const float* up_w_scales, const uint8_t* down_w_fp8, const float* down_w_scales,
                               void* bf16_output, const float* router_bias, const int32_t* expert_map,
                               cudaStream_t stream) {
  if (num_tokens > kNoAllocMaxTokens) {
    fprintf(stderr, "launch_prefill_moe_noalloc: %d tokens exceed the built-in scratch (max %d tokens)\n", num_tokens,
            kNoAllocMaxTokens);
    return -130;
  }
  unsigned char* b = nullptr;
  const int rc = noalloc_base(&b, true);
  if (rc != 0) return rc;
  return launch_prefill_moe_wgmma_q1_ep2(
      logits, num_tokens, TILE_M, b + kNaWorkspace, sizeof(Workspace), act_bf16, b + kNaActFp8,
      reinterpret_cast<float*>(b + kNaActScales), up_w_fp8, up_w_scales, down_w_fp8, down_w_scales,
      reinterpret_cast<float*>(b + kNaPartial), reinterpret_cast<int32_t*>(b + kNaTopkIds),
      reinterpret_cast<float*>(b + kNaTopkW), reinterpret_cast<int32_t*>(b + kNaSorted), bf16_output, router_bias,
      nullptr, nullptr, 0, 1, 1, 0, 0u, nullptr, nullptr, 1.0f, expert_map, stream);
}

}  // extern "C"
