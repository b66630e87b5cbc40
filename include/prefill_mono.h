/* C ABI of libprefill_mono_<variant>.so -- the drop-in boundary of the FP8 MoE prefill
 * kernel. Plain pointers and sizes only; every launch is asynchronous on the caller's
 * stream and allocates nothing. For the reference's entry points the caller owns every
 * buffer, including the workspace, and the library keeps nothing between calls except a
 * table of TMA descriptors keyed by the weights' addresses (prefill_wgmma_plan_*), the
 * wait time limit and the debug pointers set through the setters below;
 * launch_prefill_moe_noalloc alone keeps its scratch inside the library. The symbols,
 * argument order and return codes are the ones the reference's loader binds with ctypes
 * (vllm_integration/vllm/_custom_ops.py:4274-4288, :4705-4743), so its gates and its vLLM
 * quant-method hook work against this library unchanged.
 *
 * File references below are paths inside the reference repository;
 * Q  = kernel/qwen_tp/src/prefill_mono_final_nb.cu
 * EP = kernel/qwen_ep/src/prefill_mono_final_nb.cu
 *
 * Return codes of the launch entry points (Q:1569-1599, Q:1621-1638, EP:1658-1659):
 *     0      launched
 *  -100      workspace null or smaller than prefill_wgmma_workspace_bytes()
 *  -101      num_tokens <= 0
 *  -102      num_tokens*top_k/128 + local experts exceeds prefill_wgmma_max_tiles()
 *  -103      device has fewer SMs than prefill_wgmma_grid_size()
 *  -104      a required pointer is null
 *  -110..-114 fused tensor-parallel arguments (chunk count, ncomm, rank/world, pads, chunk alignment)
 *  -120      expert-parallel build called without an expert map
 *  -121      non-expert-parallel build called with an expert map
 *  -2 / -3   tensor-map encoding failed (up / down weights)
 *  > 0       cudaError_t
 * -100, -120, -121, -101, -102, -104, -110..-114 are returned, in this order of checking (EP:1650-1683),
 * before any CUDA call is made; -103 follows the query of the device's SM count, -2 / -3 / -4 the
 * descriptor encoding, -107 the cluster occupancy query. Nothing has been enqueued when a negative
 * code comes back.
 *
 * Buffers (T = num_tokens, k = top_k = 8, E = 256 routed experts, El = local experts):
 *   logits            fp32 [T, E]                      in
 *   workspace         >= prefill_wgmma_workspace_bytes(); zeroed by the launch itself
 *   act_bf16          bf16 [T, K]                      in
 *   act_fp8           u8   [T, K]                      scratch/out: e4m3 activations
 *   act_scales        fp32 [T, K/128]                  scratch/out
 *   up_w_fp8          e4m3 [El, 2*N_HALF, K]           gate rows then up rows
 *   up_w_scales       fp32 [El, 2*N_HALF/128, K/128]
 *   down_w_fp8        e4m3 [El, H, N_HALF]
 *   down_w_scales     fp32 [El, H/128, N_HALF/128]
 *   output_accum      >= T*k*H*2 bytes                 scratch: bf16 partial rows [T*k, H]
 *   topk_ids          i32  [T, k]                      out (local ids, -1 = not on this rank)
 *   topk_weights      fp32 [T, k]                      out (already renormalised)
 *   sorted_token_ids  i32  [T*k]                       out: flat slots t*k+j grouped by expert,
 *                                                      ascending inside an expert (stable)
 *   bf16_output       bf16 [T, H]                      out
 */
#ifndef PREFILL_MONO_H_
#define PREFILL_MONO_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* prefill_mono_stream_t; /* cudaStream_t */

/* ---- launch entry points ------------------------------------------------------------ */

/* Q:1726-1739. Routing from logits, no bias. */
int launch_prefill_moe_wgmma_q1(const float* logits, int num_tokens, int block_m, void* workspace,
                                size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8, float* act_scales,
                                const uint8_t* up_w_fp8, const float* up_w_scales, const uint8_t* down_w_fp8,
                                const float* down_w_scales, float* output_accum, int32_t* topk_ids,
                                float* topk_weights, int32_t* sorted_token_ids, void* bf16_output,
                                prefill_mono_stream_t stream);

/* Q:1708-1722. Adds the per-expert selection bias of the sigmoid router modes (fp32 [E] or null). */
int launch_prefill_moe_wgmma_q1_router(const float* logits, int num_tokens, int block_m, void* workspace,
                                       size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                       float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                       const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                       int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                       void* bf16_output, const float* router_bias, prefill_mono_stream_t stream);

/* Q:1686-1703. Fused tensor-parallel epilogue: tp_mc is the multicast alias of bf16_output
 * on a symmetric window, tp_pads a device array of per-rank base pointers of a separate
 * symmetric barrier window of prefill_wgmma_tp_pad_words() words, tp_seqctr a caller-owned
 * 4-byte device word zeroed once. tp_ncomm == 0 or tp_mc == null runs the ordinary kernel. */
int launch_prefill_moe_wgmma_q1_tp(const float* logits, int num_tokens, int block_m, void* workspace,
                                   size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8, float* act_scales,
                                   const uint8_t* up_w_fp8, const float* up_w_scales, const uint8_t* down_w_fp8,
                                   const float* down_w_scales, float* output_accum, int32_t* topk_ids,
                                   float* topk_weights, int32_t* sorted_token_ids, void* bf16_output,
                                   const float* router_bias, void* tp_mc, void* tp_pads, int tp_rank, int tp_world,
                                   int tp_nchunk, int tp_ncomm, uint32_t tp_seq, void* tp_seqctr,
                                   prefill_mono_stream_t stream);

/* Q:1547-1568. _tp plus a bf16 [T,H] residual folded into the same reduce and an fp32 scale
 * on the routed sum: out = bf16(out_scale * sum_k partial_k + residual). */
int launch_prefill_moe_wgmma_q1_tp2(const float* logits, int num_tokens, int block_m, void* workspace,
                                    size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                    float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                    const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                    int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                    void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                    int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                    void* tp_seqctr, const void* tp_residual, float out_scale,
                                    prefill_mono_stream_t stream);

/* EP:1809-1823. Expert parallel: expert_map is i32 [E], local slot of each global expert or -1.
 * The output is this rank's partial sum. */
int launch_prefill_moe_wgmma_q1_ep(const float* logits, int num_tokens, int block_m, void* workspace,
                                   size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8, float* act_scales,
                                   const uint8_t* up_w_fp8, const float* up_w_scales, const uint8_t* down_w_fp8,
                                   const float* down_w_scales, float* output_accum, int32_t* topk_ids,
                                   float* topk_weights, int32_t* sorted_token_ids, void* bf16_output,
                                   const float* router_bias, const int32_t* expert_map, prefill_mono_stream_t stream);

/* EP:1627-1651. The superset entry every other one forwards to. */
int launch_prefill_moe_wgmma_q1_ep2(const float* logits, int num_tokens, int block_m, void* workspace,
                                    size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                    float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                    const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                    int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                    void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                    int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                    void* tp_seqctr, const void* tp_residual, float out_scale,
                                    const int32_t* expert_map, prefill_mono_stream_t stream);

/* ---- compiled geometry and capabilities (host only, no CUDA call) -------------------- */

size_t prefill_wgmma_workspace_bytes(void);   /* Q:1515 */
int prefill_wgmma_num_experts(void);          /* Q:1516 */
int prefill_wgmma_num_experts_local(void);    /* EP:1587 */
int prefill_wgmma_ep_capable(void);           /* EP:1592 */
int prefill_wgmma_top_k(void);                /* Q:1517 */
int prefill_wgmma_max_tiles(void);            /* Q:1518 */
int prefill_wgmma_grid_size(void);            /* Q:1519; 148 here */
int prefill_wgmma_k_dim(void);                /* Q:1520 */
int prefill_wgmma_h_dim(void);                /* Q:1521 */
int prefill_wgmma_fused_renorm(void);         /* Q:1527; 1 = weights already renormalised */
int prefill_wgmma_router_mode(void);          /* Q:1741; 0 softmax, 1 sigmoid+bias, 2 grouped */
int prefill_wgmma_n_group(void);              /* Q:1742 */
int prefill_wgmma_topk_group(void);           /* Q:1743 */
int prefill_wgmma_n_up(void);                 /* Q:1748 */
int prefill_wgmma_n_half(void);               /* Q:1749 */
int prefill_wgmma_block_m(void);              /* Q:1754; rows per tile, 128 */
int prefill_wgmma_tp_max_c(void);             /* Q:1764 */
int prefill_wgmma_tp_align(void);             /* Q:1765 */
int prefill_wgmma_tp_mm(void);                /* Q:1766 */
int prefill_wgmma_tp_has_devseq(void);        /* Q:1771 */
int prefill_wgmma_tp_seq_bytes(void);         /* Q:1774 */
int prefill_wgmma_tp_has_residual(void);      /* Q:1779 */
int prefill_wgmma_tp_pad_words(int nchunk, int ncomm, int world); /* Q:1782-1784 */
int prefill_wgmma_up_pipe(void);              /* Q:1786; weight ring depth */
int prefill_wgmma_dn_pipe(void);              /* Q:1787; weight ring depth (one ring serves both phases) */
int prefill_wgmma_a_stages(void);             /* Q:1788; activation ring depth */
int prefill_wgmma_shm_total(void);            /* Q:1789 */

/* ---- additions of this library: no counterpart in the reference ---------------------- */

/* launch_prefill_moe_wgmma_q1_ep2 plus tp_peers: a device array of tp_world pointers, every rank's address of the
 * output window (the reference's symmetric pool exposes the same table, fused_moe/symm_output_pool.py:95-149; its
 * kernel does not use it). With two ranks the in-kernel reduce then reads the peer's copy directly over NVLink,
 * adds its own copy from local memory and writes the sum to both ranks: the same bits as the multicast reduce for two
 * thirds of the link traffic (through the multicast alias the switch fetches this rank's own copy over NVLink too).
 * With more ranks, or a null table, it behaves exactly like the _ep2 entry. */
int prefill_wgmma_tp_has_peer_reduce(void);   /* 1 = launch_prefill_moe_wgmma_q1_ep3 is usable */
int launch_prefill_moe_wgmma_q1_ep3(const float* logits, int num_tokens, int block_m, void* workspace,
                                    size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                    float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                    const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                    int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                    void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                    int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                    void* tp_seqctr, const void* tp_residual, float out_scale,
                                    const int32_t* expert_map, void* tp_peers, prefill_mono_stream_t stream);

/* The router linear inside the launch. The reference leaves it to the model (a separate GEMM before the
 * hook, vllm_integration/vllm/_custom_ops.py:4618 takes finished logits). router_w_bf16 is the gate weight
 * [E, K] in bf16; logits_out [T, E] fp32 receives the logits the kernel computed and routed on. The
 * arguments from num_tokens on are those of launch_prefill_moe_wgmma_q1_ep2. Every CTA computes the
 * logits of the tokens it routes itself (tcgen05.mma kind::f16, fp32 accumulation over ascending K slabs
 * of 64), so no extra grid barrier is needed. -105: router_w_bf16 or logits_out is null. */
int prefill_wgmma_has_router_gemv(void);      /* 1 = launch_prefill_moe_wgmma_q1_gemv is usable */
int launch_prefill_moe_wgmma_q1_gemv(const void* router_w_bf16, float* logits_out, int num_tokens, int block_m,
                                     void* workspace, size_t workspace_bytes, const void* act_bf16, uint8_t* act_fp8,
                                     float* act_scales, const uint8_t* up_w_fp8, const float* up_w_scales,
                                     const uint8_t* down_w_fp8, const float* down_w_scales, float* output_accum,
                                     int32_t* topk_ids, float* topk_weights, int32_t* sorted_token_ids,
                                     void* bf16_output, const float* router_bias, void* tp_mc, void* tp_pads,
                                     int tp_rank, int tp_world, int tp_nchunk, int tp_ncomm, uint32_t tp_seq,
                                     void* tp_seqctr, const void* tp_residual, float out_scale,
                                     const int32_t* expert_map, prefill_mono_stream_t stream);

/* Plan / run split (the reference rebuilds both TMA descriptors and re-sets the kernel attribute on every
 * call, Q:1611-1639, 1655; docs/FLASHINFER_UPSTREAM_NOTES.md:42-46 asks for the split). Descriptors are kept in
 * a table keyed by the tensors' addresses and found again by every later launch; the kernel's shared-memory
 * attribute is set once per device. prefill_wgmma_plan_prepare does both ahead of the first launch of a layer
 * (optional: an unprepared layer is prepared by its first launch). Returns 0, -104 (null), -2 / -3, or a
 * cudaError_t. prefill_wgmma_plan_stats reports look-ups served from the table / encoded anew;
 * prefill_wgmma_plan_reset forgets every descriptor (call it when weights are freed and their addresses may be
 * reused by tensors of another shape). */
int prefill_wgmma_plan_prepare(const uint8_t* up_w_fp8, const uint8_t* down_w_fp8);
void prefill_wgmma_plan_stats(unsigned long long* hits, unsigned long long* misses);
void prefill_wgmma_plan_reset(void);

/* The gated shared expert inside the same launch (in the reference it is a separate vLLM MLP whose output comes
 * back as tp_residual, fused_moe/runner/moe_runner.py:884-906). The argument list of the _ep2 entry, then: the
 * shared expert's block-FP8 weights in the layout of ONE routed expert (sh_up_w_fp8 e4m3 [2*N_HALF, K] gate rows then
 * up rows, sh_up_w_scales fp32 [2*N_HALF/128, K/128], sh_down_w_fp8 e4m3 [H, N_HALF], sh_down_w_scales fp32
 * [H/128, N_HALF/128]; under tensor parallelism the rank's slice, like the routed weights); sh_gate_bf16, bf16 [K] or
 * null: the expert's rows are multiplied by sigmoid(x . g), by 1 when null; sh_gate_scratch fp32 [T] (required with
 * a gate); (sh_part, sh_parts): this launch computes the shared expert for the 128-token tiles j with
 * j % sh_parts == sh_part -- expert-parallel ranks pass (rank, world), everybody else (0, 1). output_accum has to hold
 * num_tokens * (top_k + 1) * prefill_wgmma_partial_chunks() rows. Result: bf16(out_scale * routed + shared + residual).
 * -108: the two-CTA build has no shared expert; -109: a shared-expert argument is null or (sh_part, sh_parts) is not
 * a valid split; -5: descriptor encoding failed. */
int prefill_wgmma_has_shared_expert(void);    /* 1 = launch_prefill_moe_wgmma_q1_shared is usable */
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
                                       int sh_part, int sh_parts, prefill_mono_stream_t stream);

int prefill_wgmma_arch(void);                 /* 100 = built for sm_100a */
/* 1 = tiles run as pairs on clusters of two CTAs (tcgen05 cta_group::2); the total_tiles word of the
 * workspace then counts pairs, and launch_prefill_moe_wgmma_q1_gemv returns -106 (no router linear).
 * -107 from any launch: fewer than grid_size/2 two-CTA clusters can be resident on this device. */
int prefill_wgmma_cta_pair(void);
/* Chunks the intermediate is processed in: 1 up to N_HALF = 512, N_HALF/512 beyond. output_accum holds
 * num_tokens * top_k * chunks rows of H bf16 values (the reference's fp32 [T*8, H] allocation is large
 * enough for 1 or 2 chunks). */
int prefill_wgmma_partial_chunks(void);
int prefill_wgmma_block_threads(void);        /* threads per CTA */
int prefill_wgmma_stable_sort(void);          /* 1 = sorted_token_ids is deterministic (stable) */
/* Bounded waits: every device-side wait gives up after the time limit, records
 * (code << 24 | site << 16 | block) in the 32-bit status word of the workspace and the
 * launch returns normally. Read the word after synchronising; 0 = success. */
int prefill_wgmma_status_offset(void);
int prefill_wgmma_status_bytes(void);
void prefill_wgmma_set_wait_timeout_us(unsigned long long microseconds); /* later launches; default 2 s */
/* Offsets of the read-back counters inside the workspace. */
int prefill_wgmma_counts_offset(void);        /* i32 [E]   rows per local expert */
int prefill_wgmma_offsets_offset(void);       /* i32 [E+1] exclusive prefix sum */
int prefill_wgmma_total_tiles_offset(void);   /* i32 */
int prefill_wgmma_phase_ns_offset(void);      /* u64 [8] %globaltimer at phase boundaries */
int prefill_wgmma_prof_offset(void);          /* u64 [148][16] stall counters, filled only by profiling builds */
/* Debug dump targets for later launches (device pointers or null): raw gate|up sums
 * fp32 [T*k, 2*N_HALF], e4m3 intermediate [T*k, N_HALF], its scales fp32 [T*k, N_HALF/128],
 * indexed by sorted row. */
void prefill_wgmma_set_debug(void* acc, void* inter, void* inter_scale);

/* Launch that allocates nothing and needs no scratch from the caller. No counterpart in the
 * reference. For hosts that cannot obtain device memory at call time (all of HBM already given to
 * a KV-cache pool; callers that cannot take the device-wide synchronisation of cudaMalloc): the
 * workspace, the e4m3 activations, routing results, sort permutation and partial rows live in a
 * fixed array inside the library, prefill_wgmma_noalloc_scratch_bytes() per GPU for the life of
 * the process. At most prefill_wgmma_noalloc_max_tokens() tokens (256 for H = 2048, 64 for
 * H = 7168, 32 for its shards wider than 512 columns); more returns -130 and launches nothing; -131 if the array's address cannot be
 * resolved. All calls on a device share the array: calls whose kernels overlap on the GPU race,
 * so keep them ordered. The first call on each device looks the array up (cudaGetSymbolAddress);
 * make it outside stream capture. expert_map and router_bias as in the _ep entry (null when unused). */
int launch_prefill_moe_noalloc(const float* logits, int num_tokens, const void* act_bf16, const uint8_t* up_w_fp8,
                               const float* up_w_scales, const uint8_t* down_w_fp8, const float* down_w_scales,
                               void* bf16_output, const float* router_bias, const int32_t* expert_map,
                               prefill_mono_stream_t stream);
int prefill_wgmma_noalloc_max_tokens(void);
size_t prefill_wgmma_noalloc_scratch_bytes(void);
/* The four status words (status, abort flag, two detail words) of the last launch_prefill_moe_noalloc on the
 * current device, copied to out[0..3] on `stream`: that entry's workspace is inside the library, so this is how
 * its caller sees a bounded wait that gave up (out[0] == 0: success). Enqueue it behind the launch on the same
 * stream and read `out` after synchronising. -131 before the first launch on this device. */
int prefill_wgmma_noalloc_status(uint32_t* out, prefill_mono_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PREFILL_MONO_H_ */
