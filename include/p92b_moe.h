/* p92b_moe.h — C ABI of the B200 (sm_100a) MoE block for openPangu-2.0-Flash.
 *
 * Drop-in boundary: every entry point stands behind one call of the reference
 * engine's C++ operator API (include/p92/kernels.h, namespace p92::cuda) or of
 * ProjectionExecutor / Model::Impl on the MoE path; the citation beside each
 * declaration names the reference interface it replaces (paths relative to the
 * reference project).
 *
 * Conventions (same as the reference's kernel layer):
 *   - every pointer is a DEVICE pointer unless its name starts with host_;
 *   - BF16 is a raw uint16_t (include/p92/kernels.h:10);
 *   - NVFP4 = two E2M1 values per byte, even element in the low nibble, one
 *     E4M3 scale per 16 elements along K, one FP32 per-tensor scale (alpha);
 *   - calls are asynchronous on `stream` (a cudaStream_t passed as void*; NULL
 *     is the default stream) and use the CURRENT device;
 *   - the return value is a cudaError_t: 0 success, cudaErrorInvalidValue for
 *     bad arguments, cudaErrorMemoryAllocation, cudaErrorNotSupported, or the
 *     launch error reported right after the launch
 *     (cuda/nvfp4_grouped.cu:227-233,313,354-367);
 *   - *_destroy functions accept NULL and never fail
 *     (cuda/nvfp4_grouped.cu:176-177,324-326);
 *   - nothing is thread-safe: a plan carries mutable scratch, one host thread
 *     and one stream at a time per plan (src/executor.cpp:20-23).
 * Shapes: hidden and intermediate sizes are run-time arguments (multiples of
 * 64); the router is fixed at 256 experts / top-8 like the reference
 * (cuda/nvfp4_ops.cu:365-367).
 */
#ifndef P92B_MOE_H
#define P92B_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define P92B_ROUTED_EXPERTS 256
#define P92B_TOP_K 8

/* Binary-compatible with p92::cuda::Nvfp4ExpertProjection
 * (include/p92/kernels.h:12-16): three device pointers. */
typedef struct p92b_expert_projection {
    const uint8_t* weight;          /* [rows][columns/2] packed E2M1, K-major */
    const uint8_t* scales_swizzled; /* E4M3, 128x4-tiled (cuda/nvfp4_ops.cu:869-890) */
    const float* alpha;             /* device pointer to weight_scale_2 */
} p92b_expert_projection;

typedef struct p92b_bank p92b_bank; /* one layer's expert weights, retiled and owned by the library */
typedef struct p92b_plan p92b_plan; /* scratch for up to max_rows tokens; replaces Nvfp4GroupedPlan + executor scratch */

/* ---- element-wise / router operators ------------------------------------ */

/* p92::cuda::bf16_gemv_f32 (include/p92/kernels.h:121-126; cuda/nvfp4_ops.cu:161-176,1019-1030).
 * Router logits for ONE token, the reference's T=1 summation order. */
int p92b_bf16_gemv_f32(const uint16_t* input, const uint16_t* weight, float* output, int rows,
                       int columns, void* stream);

/* p92::cuda::bf16_gemm_f32 (include/p92/kernels.h:128-134; cuda/nvfp4_ops.cu:178-207,1032-1046).
 * Router logits for batch_rows tokens, the reference's T>1 summation order; output [batch_rows][rows]. */
int p92b_bf16_gemm_f32(const uint16_t* input, const uint16_t* weight, float* output, int batch_rows,
                       int rows, int columns, void* stream);

/* p92::cuda::router_top8 / router_top8_rows (include/p92/kernels.h:192-206; cuda/nvfp4_ops.cu:357-433,1160-1186). */
int p92b_router_top8(const float* logits, const float* correction_bias, int32_t* expert_ids,
                     float* expert_weights, float routed_scale, void* stream);
int p92b_router_top8_rows(const float* logits, const float* correction_bias, int32_t* expert_ids,
                          float* expert_weights, int rows, float routed_scale, void* stream);

/* p92::cuda::nvfp4_quantize (include/p92/kernels.h:479-484; cuda/nvfp4_ops.cu:818-841,1304-1315).
 * `elements` BF16 values -> elements/2 packed bytes + elements/16 linear scales. */
int p92b_nvfp4_quantize(const uint16_t* input, uint8_t* output, uint8_t* scales, int elements,
                        float global_scale, void* stream);

/* p92::cuda::nvfp4_swizzled_scale_bytes / nvfp4_swizzle_scales
 * (include/p92/kernels.h:494-502; cuda/nvfp4_ops.cu:869-890,1332-1353). */
size_t p92b_nvfp4_swizzled_scale_bytes(int rows, int scale_columns);
int p92b_nvfp4_swizzle_scales(const uint8_t* linear, uint8_t* swizzled, int rows, int scale_columns,
                              void* stream);

/* The offline weight quantiser's arithmetic (cuda/nvfp4_pack.cu:141-176,255-256):
 * per-tensor amax -> *weight_scale_2 = amax/(6*448) (device float) -> packed E2M1 + linear E4M3 scales. */
int p92b_nvfp4_pack_weight(const uint16_t* input, uint8_t* packed, uint8_t* scales, size_t elements,
                           float* weight_scale_2, void* stream);

/* The same for `matrices` equally sized tensors stored back to back (what a loader that quantises a
 * whole layer does, the per-tensor loop of cuda/nvfp4_pack.cu:235-262): per-tensor amax and scale, three launches
 * for the batch.  weight_scale_2[matrices]. */
int p92b_nvfp4_pack_weight_batch(const uint16_t* input, uint8_t* packed, uint8_t* scales, size_t elements_per_matrix,
                                 int matrices, float* weight_scale_2, void* stream);

/* p92::cuda::swiglu (include/p92/kernels.h:100-104; cuda/nvfp4_ops.cu:97-105,948-956). */
int p92b_swiglu(const uint16_t* gate, const uint16_t* up, uint16_t* output, int elements, void* stream);

/* p92::cuda::expert_combine / expert_combine_rows (include/p92/kernels.h:55-68; cuda/nvfp4_ops.cu:107-142,958-988). */
int p92b_expert_combine(const uint16_t* expert_rows, const float* route_weights, uint16_t* output,
                        int experts, int elements, void* stream);
int p92b_expert_combine_rows(const uint16_t* expert_rows, const float* route_weights, uint16_t* output,
                             int batch_rows, int experts, int elements, void* stream);

/* p92::cuda::rmsnorm (include/p92/kernels.h:77-83; cuda/nvfp4_ops.cu:67-90,907-918): the operator the engine runs
 * before (pre_mlp_norm) and after (post_mlp_norm) the MoE block, src/model.cpp:211-218,1210-1217.  Bit-exact with
 * the reference's kernel (same summation order, same fast-math rsqrtf and division).  elements <= 24576. */
int p92b_rmsnorm(const uint16_t* input, const uint16_t* weight, uint16_t* output, int rows, int elements, float epsilon,
                 void* stream);
/* p92::cuda::rmsnorm_strided (include/p92/kernels.h:85-93; cuda/nvfp4_ops.cu:920-937): rows `input_stride` /
 * `output_stride` elements apart. */
int p92b_rmsnorm_strided(const uint16_t* input, int input_stride, const uint16_t* weight, uint16_t* output,
                         int output_stride, int rows, int elements, float epsilon, void* stream);

/* p92::cuda::add_inplace (include/p92/kernels.h:95-98; cuda/nvfp4_ops.cu:92-95). */
int p92b_add_inplace(uint16_t* destination, const uint16_t* source, int elements, void* stream);

/* ---- permutation into expert-contiguous order --------------------------- */

/* Replaces the ranking loop of prepare_grouped_pointers_kernel
 * (cuda/nvfp4_grouped.cu:117-132) and the host scan of src/model.cpp:1528-1540:
 * stable counting sort of the flat index row*8+slot by expert id.
 *   order[pos] = flat index, position[flat] = pos (either may be NULL),
 *   counts[experts], offsets[experts+1] (exclusive prefix).
 * `plan` supplies the scratch and bounds `assignments` to 8*max_rows. */
int p92b_moe_permute(p92b_plan* plan, const int32_t* expert_ids, int assignments, int32_t* order,
                     int32_t* position, int32_t* counts, int32_t* offsets, void* stream);

/* Same permutation for callers that cannot allocate device memory.  No counterpart in the
 * reference: this entry point exists only in this library.
 *
 * p92b_moe_permute borrows its scratch from a plan, and a plan is a cudaMalloc.  Some hosts of
 * this code have no allocator to offer: an engine that hands its whole device-memory budget to
 * its own arena at start-up (the reference sizes its resident banks to the card and allocates
 * nothing afterwards), a plug-in loaded into a process whose policy forbids further CUDA
 * allocations, or a serving loop that must never meet the device-wide synchronisation an
 * allocation or a free can imply.  For them the scratch (per-chunk histograms and one status
 * word, P92B_STATIC_PERMUTE_SCRATCH_BYTES in all) is a fixed array inside the library image:
 * every GPU that loads the library holds it until the process exits.
 *
 * Limits and rules:
 *   - assignments <= P92B_STATIC_PERMUTE_MAX_ASSIGNMENTS (8192 rows x 8); larger requests are
 *     rejected with cudaErrorInvalidValue and a message on stderr, nothing is launched;
 *   - the call performs no cudaMalloc / cudaFree and uses no allocating library routine;
 *   - the first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress with that device current) and remembers it; make that first call
 *     before starting any stream capture on that device;
 *   - all calls on a device share the one array, which still holds the previous call's contents:
 *     the entry point clears the status word and its scan's block counter itself and overwrites
 *     every histogram it reads, but
 *     two calls whose kernels overlap on the GPU (different streams) race and must be serialised
 *     by the caller;
 *   - outputs as p92b_moe_permute: order/position may be NULL, counts[256], offsets[257]. */
#define P92B_STATIC_PERMUTE_MAX_ASSIGNMENTS 65536
#define P92B_STATIC_PERMUTE_SCRATCH_BYTES (P92B_STATIC_PERMUTE_MAX_ASSIGNMENTS / 256 * 256 * 4 + 256)
int p92b_moe_permute_static(const int32_t* expert_ids, int assignments, int32_t* order, int32_t* position,
                            int32_t* counts, int32_t* offsets, void* stream);
/* Status of the p92b_moe_permute_static calls made so far on `stream` of the current device (no
 * counterpart in the reference).  An expert id outside 0..255 does not fault: it is counted as
 * expert 0 or 255 and the call records 1 in a status word that sits in the same built-in array,
 * out of the caller's reach; a caller without a plan has no p92b_plan_get_views to read it through.
 * This copies the word of the most recent call into *host_status (0 = every id was in range) and
 * synchronises `stream`; it allocates nothing either.  Each permutation call clears the word when it
 * starts, so ask before issuing the next one.
 * Host threads: the first call on a device by either entry point looks the array up; two threads
 * doing that at once is harmless, but their kernels would share the array, so they must be
 * serialised all the same. */
int p92b_moe_permute_static_status(int32_t* host_status, void* stream);

/* ---- expert bank --------------------------------------------------------- */

/* Replaces the expert-table build of Model::Impl::bind_weights (src/model.cpp:772-805)
 * and the ResidentProjection layout of src/resident.cpp:75-162.
 * host_entries: HOST array of (local_experts + 1) * 3 entries in the reference's
 * bank order expert*3 + kind, kind 0/1/2 = gate/up/down (cuda/nvfp4_grouped.cu:133);
 * the last three entries are the shared expert.  The weights are copied into
 * the library's own layout - a tile stream in which the bytes of every pipeline stage of the
 * tensor-core kernels are contiguous ("retiled for TMA") - and the caller may free its copies
 * afterwards.  flags: reserved, pass 0.
 * first_expert / local_experts select the expert-parallel shard this bank holds
 * (0 / 256 on one GPU); local_experts = 0 makes a bank of one entry for p92b_dense_forward. */
int p92b_bank_create(p92b_bank** bank, const p92b_expert_projection* host_entries, int first_expert,
                     int local_experts, int hidden, int intermediate, int flags, void* stream);
void p92b_bank_destroy(p92b_bank* bank);
size_t p92b_bank_bytes(const p92b_bank* bank);

/* ---- weight container ("P92FP41") and resident loading ----------------------------------------------- */

/* Replaces p92::Nvfp4Artifact (include/p92/nvfp4_artifact.h:36-71; src/nvfp4_artifact.cpp:65-146): read-only maps
 * of manifest.bin (48-byte header + 128-byte records sorted by name), weights.nvfp4, scales.e4m3 and, if present,
 * scales.swizzled.e4m3, with the reference reader's checks (magic, version, record size, file sizes, name order,
 * rows % 128, columns % 16, weight_scale_2 > 0, extents inside the files).  Where the reference throws, these
 * return cudaErrorInvalidValue (cudaErrorFileNotFound for a missing file) and keep the reference's message text for
 * p92b_artifact_last_error (per thread).  Host side only: no GPU is needed to open and query a container. */
typedef struct p92b_artifact p92b_artifact;
typedef struct p92b_artifact_record {      /* binary layout of p92::Nvfp4Record (include/p92/nvfp4_artifact.h:24-32) */
    char name[96];
    uint32_t rows;
    uint32_t columns;
    uint64_t weight_offset;
    uint64_t scale_offset;
    float weight_scale_2;
    uint32_t reserved;
} p92b_artifact_record;
int p92b_artifact_open(p92b_artifact** artifact, const char* directory);
void p92b_artifact_close(p92b_artifact* artifact);
int p92b_artifact_tensor_count(const p92b_artifact* artifact);
int p92b_artifact_has_swizzled_scales(const p92b_artifact* artifact);
int p92b_artifact_at(const p92b_artifact* artifact, int index, p92b_artifact_record* record);
int p92b_artifact_find(const p92b_artifact* artifact, const char* name, p92b_artifact_record* record);
const uint8_t* p92b_artifact_weight(const p92b_artifact* artifact, const p92b_artifact_record* record);   /* host pointers */
const uint8_t* p92b_artifact_scales(const p92b_artifact* artifact, const p92b_artifact_record* record);
const char* p92b_artifact_last_error(void);

/* Replaces ResidentWeights::open + find (src/resident.cpp:75-162) and the table build of Model::Impl::bind_weights
 * (src/model.cpp:667-681,724,772-805) for ONE layer: uploads the layer's routed experts first_expert ..
 * first_expert + local_experts - 1 ("model.layers.<l>.mlp.experts.<e>.{gate,up,down}_proj.weight") and its shared
 * expert ("...mlp.shared_experts...") and retiles them straight into a bank.  Scales are taken from
 * scales.swizzled.e4m3 when the container has it, else tiled on the device, as the reference does.  The staging
 * copies are freed before the call returns; the bank holds the only resident copy. */
int p92b_bank_create_from_artifact(p92b_bank** bank, const p92b_artifact* artifact, int layer_index, int first_expert,
                                   int local_experts, void* stream);
/* The same for the dense MLP of layers 0-1 ("model.layers.<l>.mlp.{gate,up,down}_proj.weight", src/model.cpp:720):
 * a bank of one entry for p92b_dense_forward. */
int p92b_dense_bank_create_from_artifact(p92b_bank** bank, const p92b_artifact* artifact, int layer_index, void* stream);

/* ---- plan + whole block -------------------------------------------------- */

/* Replaces nvfp4_grouped_plan_create/_destroy (include/p92/kernels.h:25-30) and
 * ProjectionExecutor::reserve (src/executor.cpp:109-140): all scratch is sized
 * once for max_rows, so no call on the hot path allocates or synchronises. */
int p92b_plan_create(p92b_plan** plan, int max_rows, int hidden, int intermediate);
void p92b_plan_destroy(p92b_plan* plan);
size_t p92b_plan_bytes(const p92b_plan* plan);

/* Replaces Model::Impl::run_moe (src/model.cpp:1677-1729) and run_moe_rows
 * (src/model.cpp:1486-1573): router logits -> top-8 -> permutation -> NVFP4
 * gate/up + SwiGLU -> NVFP4 down -> weighted combine (device law,
 * cuda/nvfp4_ops.cu:124-142) -> + shared expert.  input/output: BF16 [rows][hidden].
 * rows == 1 uses the T=1 logits order, rows > 1 the T>1 order, as the reference does.  From 9 rows on the logits
 * are a BF16 tensor-core product and only the ones that can decide the top-8 (every expert within a proven error bound
 * of the 8th best, about nine per token) are recomputed in the reference's exact order; expert ids and route weights
 * are still the reference's bit for bit, the `logits` view then holds approximate values except at those positions.
 * P92B_EXACT_LOGITS=1 in the environment keeps the exact-order kernel at every size.
 *
 * For up to 16 rows the block is ONE persistent kernel with one thread block per SM whose blocks hand
 * data to one another (p92b_plan_set_path).  They must all be resident at once: do not run it while
 * kernels on other streams keep SMs occupied for long.  Every wait inside is bounded: if the blocks cannot
 * make progress within about a second the call ends with 2 in the plan's status word (p92b_plan_get_views)
 * instead of hanging.  The same holds for p92b_ep_forward_fused. */
int p92b_moe_forward(p92b_plan* plan, const p92b_bank* bank, const uint16_t* input,
                     const uint16_t* router_weight, const float* correction_bias, uint16_t* output,
                     int rows, float routed_scale, void* stream);

/* The block with the two RMSNorms the engine runs either side of it (src/model.cpp:211-218 decode, :1210-1217
 * prefill rows): output = rmsnorm(block(rmsnorm(input, pre_norm_weight)), post_norm_weight), each norm the reference's
 * operator bit for bit (p92b_rmsnorm), so the routing equals the reference's on the same `mixed_` rows.  Either weight
 * may be NULL (that norm is skipped); norm_epsilon is the engine's kNormEpsilon (src/model.cpp:57).  For up to 16 rows
 * both norms run inside the one persistent kernel - the pre-norm where it stages the token rows, the post-norm behind
 * its combine - so the engine saves two launches per layer; larger batches run p92b_rmsnorm around the pipeline. */
int p92b_moe_forward_normed(p92b_plan* plan, const p92b_bank* bank, const uint16_t* input, const uint16_t* pre_norm_weight,
                            const uint16_t* post_norm_weight, float norm_epsilon, const uint16_t* router_weight,
                            const float* correction_bias, uint16_t* output, int rows, float routed_scale, void* stream);

/* Replaces Model::Impl::run_dense / run_dense_rows (src/model.cpp:1476-1484,1668-1675), the dense SwiGLU MLP of
 * layers 0-1 (intermediate 9216): output = down(bf16 swiglu(gate(x), up(x))), each projection the quantise + NVFP4
 * product of ProjectionExecutor::project_rows (src/executor.cpp:148-179).  It runs on the grouped tcgen05 kernels as
 * a bank with no routed experts: create the bank with local_experts = 0 and the MLP's gate/up/down as its only
 * three entries (p92b_bank_create), the plan with the MLP's intermediate size.  Same rounding chain as an expert:
 * x -> FP4; gate, up -> BF16; SwiGLU -> BF16 -> FP4; down -> BF16. */
int p92b_dense_forward(p92b_plan* plan, const p92b_bank* bank, const uint16_t* input, uint16_t* output, int rows,
                       void* stream);

/* Same block, HOST input and output buffers (pinned or pageable): copies the
 * rows in, runs p92b_moe_forward, copies the result out and synchronises the
 * stream.  The call a host-resident caller makes. */
int p92b_moe_forward_host(p92b_plan* plan, const p92b_bank* bank, const uint16_t* host_input,
                          const uint16_t* router_weight, const float* correction_bias,
                          uint16_t* host_output, int rows, float routed_scale, void* stream);
/* The same as a pipeline for a loop over layers: nothing is synchronised, the block is enqueued on
 * `stream`, and the two copies run on two streams of the plan's own, so that the rows of one call travel
 * while the blocks of its neighbours compute (two sets of staging rows, used alternately).  The two host
 * buffers must be page-locked; the input must hold its data when the call is made (it is read by a stream
 * that is not ordered after `stream`); both must stay valid, and the output may be read, once
 * p92b_plan_host_flush(plan, stream) has been called and `stream` synchronised: the flush makes `stream`
 * wait for the copies still going out.  One plan, one thread. */
int p92b_moe_forward_host_async(p92b_plan* plan, const p92b_bank* bank, const uint16_t* pinned_input,
                                const uint16_t* router_weight, const float* correction_bias, uint16_t* pinned_output,
                                int rows, float routed_scale, void* stream);
int p92b_plan_host_flush(p92b_plan* plan, void* stream);

/* Stage entry points at the reference's split, so each existing call can be replaced alone.  Both run on the
 * grouped tcgen05 kernels from the same bank as the whole-block call (an epilogue that stores BF16 gate and up
 * un-fused; the down product writing the caller's (row, slot) rows), at any row count the plan holds.
 * ProjectionExecutor::project_expert_gate_up (include/p92/executor.h:31-38; src/executor.cpp:39-71):
 * gate_output / up_output BF16 [rows][8][intermediate] in (row, slot) order. */
int p92b_project_expert_gate_up(p92b_plan* plan, const p92b_bank* bank, const int32_t* expert_ids,
                                const uint16_t* input, uint16_t* gate_output, uint16_t* up_output,
                                int rows, void* stream);
/* ProjectionExecutor::project_expert_down (include/p92/executor.h:39-45; src/executor.cpp:73-107):
 * input_rows BF16 [rows*8][intermediate], output_rows BF16 [rows*8][hidden], (row, slot) order. */
int p92b_project_expert_down(p92b_plan* plan, const p92b_bank* bank, const int32_t* expert_ids,
                             const uint16_t* input_rows, uint16_t* output_rows, int rows, void* stream);

/* Stand-ins for the reference's grouped-projection plan and call, argument for argument
 * (nvfp4_grouped_plan_create / _destroy, include/p92/kernels.h:25-30; nvfp4_grouped_m1 / nvfp4_grouped_rows,
 * :32-53; cuda/nvfp4_grouped.cu:223-374), for callers that hold rows they quantised themselves and a device table of
 * Nvfp4ExpertProjection entries (tests/moe_forward_test.cpp:209-221,258-272; src/executor.cpp:60-70,96-106):
 *   - the plan is created for `groups` problems of a [rows x columns] matrix: groups = batch_rows * 16 for the gate
 *     and up pair (first_output, second_output, projection_kind 0), batch_rows * 8 for one matrix (second_output
 *     NULL; projection_kind 0, 1 or 2 = gate, up, down);
 *   - packed_input / input_scales_swizzled: the caller's NVFP4 rows and their 128x4-tiled scales, one row per token
 *     (expert_distinct_input_rows 0: the 8 slots of a token share it) or one per (token, slot) (1);
 *   - expert_bank: DEVICE array, entry expert * 3 + kind, read IN PLACE (matrices row-major, 16-byte aligned, scales
 *     128x4-tiled): no bank has to be built, no copy of the weights is made;
 *   - outputs BF16 [batch_rows * 8][rows] in (token, slot) order, bf16(alpha * product) like the reference's epilogue.
 * Rows that share an expert share its weight stream (the reference runs one N=1 problem per (token, slot)); the
 * results are the same numbers.  The reference caps batch_rows at 4 (include/p92/executor.h:61-62); here any
 * groups / 8 rows.  rows % 128 == 0, columns % 256 == 0.  Errors as cuda/nvfp4_grouped.cu:227-233,354-359; a matrix
 * pointer that is not 16-byte aligned ends the kernel with 3 in the status word (p92b_nvfp4_grouped_plan_status). */
typedef struct p92b_grouped_plan p92b_grouped_plan;
int p92b_nvfp4_grouped_plan_create(p92b_grouped_plan** plan, int groups, int rows, int columns);
void p92b_nvfp4_grouped_plan_destroy(p92b_grouped_plan* plan);
int p92b_nvfp4_grouped_m1(p92b_grouped_plan* plan, const uint8_t* packed_input, const uint8_t* input_scales_swizzled,
                          const p92b_expert_projection* expert_bank, const int32_t* expert_ids, uint16_t* first_output,
                          uint16_t* second_output, int projection_kind, int distinct_input_rows, void* stream);
int p92b_nvfp4_grouped_rows(p92b_grouped_plan* plan, const uint8_t* packed_input, const uint8_t* input_scales_swizzled,
                            const p92b_expert_projection* expert_bank, const int32_t* expert_ids, uint16_t* first_output,
                            uint16_t* second_output, int projection_kind, int batch_rows, int expert_distinct_input_rows,
                            void* stream);
int p92b_nvfp4_grouped_plan_status(const p92b_grouped_plan* plan, const int32_t** device_status);

/* ---- expert parallelism -------------------------------------------------- */
/* No counterpart in the reference (its CUDA backend is single-device, src/executor.cpp:20-23);
 * these are the device-side halves of the block either side of the two all-to-all exchanges that
 * the host issues (NCCL).  Experts are sharded contiguously: the bank of GPU g holds experts
 * [g*256/G, (g+1)*256/G) and the shared expert (p92b_bank_create first_expert/local_experts).
 *
 * p92b_ep_route: logits, top-8, stable permutation and quantisation of the local `rows`; writes the
 * 8*rows quantised rows (p92b_ep_row_bytes each: packed values then linear scales) in permuted
 * order, which is grouped by destination GPU.  counts[256] (plan views) give the split sizes.
 * p92b_ep_experts: `total_rows` arrived rows, the runs of sources 0..sources-1 concatenated, each run
 * ordered by local expert; recv_counts[sources][local_experts] (device) are the run lengths.  Places
 * them in global stable order per expert, runs gate/up + SwiGLU + down on the local shard, writes the
 * BF16 down rows [total_rows][hidden] in arrival order.  `plan` must hold max_rows >= total_rows/8.
 * p92b_ep_combine: on the home GPU, `returned_rows` [8*rows][hidden] in the order p92b_ep_route
 * produced; computes the shared expert for the local tokens (scratch from `shared_plan`) and the
 * weighted combine in slot order. */
size_t p92b_ep_row_bytes(int hidden);
int p92b_ep_route(p92b_plan* plan, const uint16_t* input, const uint16_t* router_weight,
                  const float* correction_bias, int rows, float routed_scale, uint8_t* send_rows, void* stream);
int p92b_ep_experts(p92b_plan* plan, const p92b_bank* bank, const uint8_t* recv_rows, const int32_t* recv_counts,
                    int sources, int total_rows, uint16_t* out_rows, void* stream);
int p92b_ep_combine(p92b_plan* home_plan, p92b_plan* shared_plan, const p92b_bank* bank, const uint16_t* input,
                    const uint16_t* returned_rows, uint16_t* output, int rows, void* stream);

/* The same three halves for small batches with FIXED-CAPACITY exchange blocks, so that no split size
 * ever crosses to the host and a whole layer stays asynchronous: every (source, destination) pair
 * owns one block of p92b_ep_fixed_block_bytes = header (the source's row counts for the
 * destination's experts) + cap_rows row slots; both all-to-alls have equal splits.  cap_rows must be
 * the same on all GPUs and at least 8 * rows.  send_blocks / recv_blocks: [world][block];
 * out_slots / returned_slots: BF16 [world][cap_rows][hidden]. */
size_t p92b_ep_fixed_block_bytes(int hidden, int local_experts, int cap_rows);
int p92b_ep_route_fixed(p92b_plan* plan, const uint16_t* input, const uint16_t* router_weight,
                        const float* correction_bias, int rows, float routed_scale, uint8_t* send_blocks, int world,
                        int cap_rows, void* stream);
int p92b_ep_experts_fixed(p92b_plan* plan, const p92b_bank* bank, const uint8_t* recv_blocks, int sources, int cap_rows,
                          uint16_t* out_slots, void* stream);
int p92b_ep_combine_fixed(p92b_plan* home_plan, p92b_plan* shared_plan, const p92b_bank* bank, const uint16_t* input,
                          const uint16_t* returned_slots, uint16_t* output, int rows, void* stream);

/* Small batches, fused: the whole expert-parallel block as ONE kernel launch per GPU, both exchanges
 * done by the kernel with stores into the peers' memory over NVLink (no NCCL call, no host
 * synchronisation).  Dispatch is an all-gather of the quantised token rows and their expert ids -
 * with at most 32 tokens in flight every GPU can hold the whole batch and run the single-GPU law on
 * its own experts - and the down product's epilogue places each result row directly into its home
 * GPU's window; the home GPU combines in slot order and adds its shared expert.  No counterpart in the
 * reference (one device, src/executor.cpp:20-23); the per-expert row order and the combine law are the
 * single-device ones (cuda/nvfp4_grouped.cu:117-132, cuda/nvfp4_ops.cu:124-142).
 *
 * A window is this GPU's exchange memory (p92b_ep_window_bytes, allocated with cudaMalloc) plus the
 * mapped windows of its peers; it serves this call (world * rows_per_gpu <= 32, rows_per_gpu <= 8) and
 * p92b_ep_forward_gathered below (rows_per_gpu <= 512, world * rows_per_gpu <= 1024).  Set-up, once: every process creates its window, publishes the 64-byte
 * inter-process handle (p92b_ep_window_handle) to all others by any means, and connects with the
 * handles of all ranks in rank order (its own entry is ignored).  world * rows_per_gpu <= 32,
 * rows_per_gpu <= 8.  All GPUs must call p92b_ep_forward_fused the same number of times on a window,
 * in the same order (the flags carry the call number); rows may differ per GPU and per call.  One
 * window serves any number of layers.  The plan must have been created for at least
 * world * rows_per_gpu rows.  A peer that never arrives ends the kernel after about a second with
 * status 2 (a bounded wait gave up) in the plan's status word; the window is then out of step and must be
 * recreated on all GPUs.  P92B_EP_WIDE=1 in the environment forces the 32-token variant of the kernel
 * (otherwise chosen when world * rows_per_gpu > 16). */
typedef struct p92b_ep_window p92b_ep_window;
int p92b_ep_window_create(p92b_ep_window** out, int rank, int world, int rows_per_gpu);
void p92b_ep_window_destroy(p92b_ep_window* window);
size_t p92b_ep_window_bytes(const p92b_ep_window* window);
int p92b_ep_window_handle(const p92b_ep_window* window, uint8_t* handle64);
int p92b_ep_window_connect(p92b_ep_window* window, const uint8_t* handles /* [world][64] */);
/* The same for windows that live in THIS process (one process driving several GPUs with peer access
 * enabled, or tests): all_windows[r] is rank r's window. */
int p92b_ep_window_connect_local(p92b_ep_window* window, p92b_ep_window* const* all_windows);
int p92b_ep_forward_fused(p92b_plan* plan, const p92b_bank* bank, p92b_ep_window* window, const uint16_t* input,
                          const uint16_t* router_weight, const float* correction_bias, uint16_t* output, int rows,
                          float routed_scale, void* stream);

/* The same with page-locked HOST rows in and out, pipelined like p92b_moe_forward_host_async (copies on the
 * plan's own two streams, two sets of staging rows; p92b_plan_host_flush + a synchronisation of `stream`
 * before the outputs are read). */
int p92b_ep_forward_fused_host_async(p92b_plan* plan, const p92b_bank* bank, p92b_ep_window* window,
                                     const uint16_t* pinned_input, const uint16_t* router_weight,
                                     const float* correction_bias, uint16_t* pinned_output, int rows, float routed_scale,
                                     void* stream);

/* Medium batches (tens of tokens per GPU, up to 1024 in flight), same idea, several launches: every GPU
 * stores its quantised rows and top-8 ids into every peer's window (all-gather), ranks the rows of its own
 * experts over the whole batch by the reference's permutation law, computes them with the grouped
 * tcgen05 kernels, stores each result row into its home GPU's window, and the home GPU combines in slot
 * order and adds its shared expert.  No NCCL call, no host synchronisation, nothing but bounded polls of
 * {payload, call number} words between GPUs.  Same window and calling rules as p92b_ep_forward_fused
 * (both kinds of call may be mixed on one window as long as all GPUs mix them identically); the plan
 * must have been created for at least world * rows_per_gpu rows. */
int p92b_ep_forward_gathered(p92b_plan* plan, const p92b_bank* bank, p92b_ep_window* window, const uint16_t* input,
                             const uint16_t* router_weight, const float* correction_bias, uint16_t* output, int rows,
                             float routed_scale, void* stream);

/* Large batches (hundreds to thousands of tokens per GPU): the same two exchanges - all-gather of the quantised
 * rows and ids, direct placement of the result rows - as plain 16-byte peer stores with one flag word per peer and
 * exchange (system-scope release / bounded acquire poll) instead of tagged words, around the grouped tcgen05
 * kernels and the large-batch router.  No collective library, no split sizes crossing to the host, no host
 * synchronisation: the whole layer is asynchronous on `stream`.  Every GPU runs the permutation law over the ids of
 * the whole batch restricted to its own experts (cuda/nvfp4_grouped.cu:117-132), and the home GPU combines in slot
 * order (cuda/nvfp4_ops.cu:124-142), so ids, per-expert row order and the combine are the single-device ones.
 * The window is created with p92b_ep_window_create_bulk (world * rows_per_gpu * 1.5 KB + rows_per_gpu * 40 KB of
 * exchange memory), published and connected like the other windows, and serves only this call; rows may differ per
 * GPU and per call (rows <= rows_per_gpu), the plan must hold world * rows_per_gpu rows.  Same calling rule: all
 * GPUs make the same sequence of calls on their windows; a peer that never arrives ends the wait after about a
 * second with status 2. */
int p92b_ep_window_create_bulk(p92b_ep_window** out, int rank, int world, int rows_per_gpu, int hidden);
int p92b_ep_forward_bulk(p92b_plan* plan, const p92b_bank* bank, p92b_ep_window* window, const uint16_t* input,
                         const uint16_t* router_weight, const float* correction_bias, uint16_t* output, int rows,
                         float routed_scale, void* stream);

/* Device views of the last p92b_moe_forward's intermediates, for tests and
 * tracing (the reference keeps the same buffers as Model::Impl members,
 * src/model.cpp:872-885).  Valid until the next call on the plan. */
typedef struct p92b_plan_views {
    const float* logits;          /* [rows][256] */
    const int32_t* expert_ids;    /* [rows][8] */
    const float* expert_weights;  /* [rows][8] */
    const int32_t* order;         /* [rows*8] */
    const int32_t* position;      /* [rows*8] */
    const int32_t* counts;        /* [256] */
    const int32_t* offsets;       /* [257] */
    const uint16_t* mixed;        /* BF16 down outputs [mixed rows][hidden] */
    const int32_t* mixed_index;   /* [rows*8 + rows]: row of `mixed` holding assignment (row, slot), then the shared rows */
    const int32_t* status;        /* device int: 0 ok, else the first error a kernel recorded: 1 expert id out of range (clamped), 2 a bounded wait gave up,
                                     3 a matrix of a caller's projection table is not 16-byte aligned */
    const int32_t* router_stats;  /* [2] large-batch router (tensor-core logits + exact repair): logits recomputed in the
                                     reference's order so far on this plan, tokens whose whole row was recomputed */
    const unsigned long long* trace; /* [trace_blocks][64] %globaltimer stamps of the last fused decode launch
                                        (written only when P92B_TRACE is set in the environment) */
    int trace_blocks;
} p92b_plan_views;
int p92b_plan_get_views(const p92b_plan* plan, p92b_plan_views* views);

/* Stage timing for measurement harnesses (the reference brackets its dispatches with CUDA
 * events the same way, tests/moe_forward_test.cpp:306-326).  While enabled, p92b_moe_forward
 * records an event pair on `stream` around every stage, synchronises the stream at the end of
 * the call and accumulates the elapsed times; off by default and free when off.
 * Stages: 0 router logits, 1 top-8, 2 permutation, 3 activation quantise, 4 gate/up + SwiGLU,
 * 5 down, 6 combine + shared add.  host_ms[7] receives the sums since enabling, host_calls the
 * number of forwards accumulated.  The multi-kernel expert-parallel calls honour it too, with their own meaning of the
 * seven slots: p92b_ep_forward_bulk 0 router, 1 dispatch (stores + wait for every peer's rows), 2 permutation +
 * placement, 3 unused, 4 gate/up, 5 down, 6 return + combine; p92b_ep_forward_gathered 0 router, 1 push, 2 routing
 * lists (waits for all ids), 3 placement (waits for all rows), 4 gate/up, 5 down, 6 return + combine. */
#define P92B_STAGES 7
int p92b_plan_stage_timing(p92b_plan* plan, int enable);
int p92b_plan_stage_times(const p92b_plan* plan, float* host_ms, int* host_calls);

/* Kernel family for the block: 0 automatic (3 for up to 16 rows, else 2), 2 tcgen05 block-scaled MMA kernels
 * (TMA + TMEM), one launch per stage, at any size, 3 the whole block as one persistent tcgen05 kernel (up to 16
 * rows).  The environment variable P92B_PATH sets the default of new plans.  Both implement the same
 * arithmetic contract. */
int p92b_plan_set_path(p92b_plan* plan, int path);

/* Number of kernels the last p92b_moe_forward on this plan launched. */
int p92b_plan_last_launches(const p92b_plan* plan);

const char* p92b_version(void);

#ifdef __cplusplus
}
#endif

#endif /* P92B_MOE_H */
