// C ABI: expert bank, plan, whole-block forward and the stage entry points.
// Host-side orchestration only; every kernel lives in the other .cu files.
#include "p92b_common.cuh"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <new>
#include <vector>

using namespace p92b;

namespace {

constexpr std::size_t kAlign = 256;

std::size_t align_up(std::size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// Carves aligned regions out of one allocation.
struct Carver {
    std::uint8_t* base = nullptr;
    std::size_t used = 0;
    template <class T>
    T* take(std::size_t count) {
        T* p = base == nullptr ? nullptr : reinterpret_cast<T*>(base + used);
        used += align_up(count * sizeof(T));
        return p;
    }
};

struct BankLayout {
    std::size_t g13, g2, alpha, total;
};

BankLayout bank_layout(int entries, int hidden, int inter) {
    BankLayout l {};
    Carver c;
    const std::size_t e = static_cast<std::size_t>(entries);
    l.g13 = c.used; c.take<std::uint8_t>(e * (inter / 128) * (hidden / 256) * kChunkBytes);
    l.g2 = c.used; c.take<std::uint8_t>(e * (hidden / 128) * (inter / 512) * kChunkBytes);
    l.alpha = c.used; c.take<float>(e * 3);
    l.total = c.used;
    return l;
}

bool shapes_match(const p92b_plan* plan, const p92b_bank* bank) {
    return plan->hidden == bank->view.hidden && plan->intermediate == bank->view.intermediate;
}

}  // namespace

extern "C" {

const char* p92b_version(void) { return "p92b-moe 0.1 (sm_100a)"; }

int p92b_bank_create(p92b_bank** out, const p92b_expert_projection* host_entries, int first_expert,
                     int local_experts, int hidden, int intermediate, int flags, void* stream_) {
    if (out == nullptr) return cudaErrorInvalidValue;
    *out = nullptr;
    if (host_entries == nullptr || first_expert < 0 || local_experts < 0 ||
        first_expert + local_experts > kExperts || hidden <= 0 || intermediate <= 0 || hidden % 256 != 0 ||
        intermediate % 512 != 0 || flags != 0) {
        return cudaErrorInvalidValue;
    }
    const int entries = local_experts + 1;
    for (int i = 0; i < entries * 3; ++i) {
        if (host_entries[i].weight == nullptr || host_entries[i].scales_swizzled == nullptr ||
            host_entries[i].alpha == nullptr) {
            return cudaErrorInvalidValue;
        }
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    p92b_bank* bank = new (std::nothrow) p92b_bank();
    if (bank == nullptr) return cudaErrorMemoryAllocation;
    const BankLayout l = bank_layout(entries, hidden, intermediate);
    cudaError_t st = cudaMalloc(&bank->storage, l.total);
    if (st != cudaSuccess) {
        delete bank;
        return cudaErrorMemoryAllocation;
    }
    bank->bytes = l.total;
    std::uint8_t* base = static_cast<std::uint8_t*>(bank->storage);
    std::uint8_t* g13 = base + l.g13;
    std::uint8_t* g2 = base + l.g2;
    float* alpha = reinterpret_cast<float*>(base + l.alpha);

    const std::size_t g13_entry = static_cast<std::size_t>(intermediate / 128) * (hidden / 256) * kChunkBytes;
    const std::size_t g2_entry = static_cast<std::size_t>(hidden / 128) * (intermediate / 512) * kChunkBytes;
    p92b_expert_projection* device_table = nullptr;
#define BANK_TRY(call)            \
    do {                          \
        st = (call);              \
        if (st != cudaSuccess) {  \
            cudaFree(device_table); \
            cudaFree(bank->storage); \
            delete bank;          \
            return st;            \
        }                         \
    } while (0)
    // the caller's table goes to the device once; three launches (one per matrix kind) then retile every
    // entry and pick up its alpha, instead of a launch and a copy per matrix
    const std::size_t table_bytes = static_cast<std::size_t>(entries) * 3 * sizeof(p92b_expert_projection);
    BANK_TRY(cudaMalloc(&device_table, table_bytes));
    BANK_TRY(cudaMemcpyAsync(device_table, host_entries, table_bytes, cudaMemcpyHostToDevice, stream));
    BANK_TRY(launch_retile_table(device_table, entries, 0, g13, g13_entry, intermediate, hidden / 2, 1, 0, alpha, stream));
    BANK_TRY(launch_retile_table(device_table, entries, 1, g13, g13_entry, intermediate, hidden / 2, 1, 1, alpha, stream));
    BANK_TRY(launch_retile_table(device_table, entries, 2, g2, g2_entry, hidden, intermediate / 2, 2, 0, alpha, stream));
    BANK_TRY(cudaStreamSynchronize(stream));
#undef BANK_TRY
    cudaFree(device_table);
    bank->view.g13 = g13;
    bank->view.g2 = g2;
    bank->view.alpha = alpha;
    bank->view.first_expert = first_expert;
    bank->view.local_experts = local_experts;
    bank->view.hidden = hidden;
    bank->view.intermediate = intermediate;
    bank->tc_ready = true;
    *out = bank;
    return cudaSuccess;
}

void p92b_bank_destroy(p92b_bank* bank) {
    if (bank == nullptr) return;
    if (bank->storage != nullptr) cudaFree(bank->storage);
    delete bank;
}

size_t p92b_bank_bytes(const p92b_bank* bank) { return bank == nullptr ? 0 : bank->bytes; }

int p92b_plan_create(p92b_plan** out, int max_rows, int hidden, int intermediate) {
    if (out == nullptr) return cudaErrorInvalidValue;
    *out = nullptr;
    if (max_rows <= 0 || max_rows > (1 << 20) || hidden <= 0 || intermediate <= 0 || hidden % 128 != 0 ||
        intermediate % 128 != 0) {
        return cudaErrorInvalidValue;
    }
    p92b_plan* plan = new (std::nothrow) p92b_plan();
    if (plan == nullptr) return cudaErrorMemoryAllocation;
    plan->max_rows = max_rows;
    plan->hidden = hidden;
    plan->intermediate = intermediate;
    int device = 0;
    cudaError_t st = cudaGetDevice(&device);
    if (st == cudaSuccess) st = cudaDeviceGetAttribute(&plan->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (st != cudaSuccess) {
        delete plan;
        return st;
    }
    const std::size_t rows = static_cast<std::size_t>(max_rows);
    plan->chunks = static_cast<int>((rows * kTop + 255) / 256);
    {
        // worst case of the padded position space: every active entry wastes (align - 1) rows
        const std::size_t align = static_cast<std::size_t>(tc_pad_align(max_rows));
        const std::size_t active = std::min<std::size_t>(kExperts, rows * kTop) + 1;
        plan->pp_rows = (rows * (kTop + 1) + active * (align - 1) + 127) / 128 * 128;
    }
    if (const char* env = std::getenv("P92B_PATH")) plan->path = std::atoi(env);
    plan->trace_on = std::getenv("P92B_TRACE") != nullptr;
    for (int pass = 0; pass < 2; ++pass) {
        Carver c;
        c.base = static_cast<std::uint8_t*>(plan->storage);
        plan->logits = c.take<float>(rows * kExperts);
        plan->ids = c.take<std::int32_t>(rows * kTop);
        plan->route_weights = c.take<float>(rows * kTop);
        plan->order = c.take<std::int32_t>(rows * kTop);
        plan->position = c.take<std::int32_t>(rows * kTop);
        plan->counts = c.take<std::int32_t>(kExperts + 1);
        plan->offsets = c.take<std::int32_t>(kExperts + 2);
        plan->row_token = c.take<std::int32_t>(rows * (kTop + 1));
        plan->active = c.take<std::int32_t>(kExperts + 1);
        plan->active_count = c.take<std::int32_t>(1);
        plan->pp_off = c.take<std::int32_t>(kExperts + 2);
        plan->tile_prefix = c.take<std::int32_t>(kExperts + 2);
        plan->tile_prefix_wide = c.take<std::int32_t>(kExperts + 2);
        plan->pp_of_flat = c.take<std::int32_t>(rows * (kTop + 1));
        plan->chunk_hist = c.take<std::int32_t>(static_cast<std::size_t>(plan->chunks) * kExperts);
        plan->scan_blocks_done = c.take<unsigned>(1);
        plan->xq = c.take<std::uint8_t>(rows * (hidden / 2));
        plan->xs = c.take<std::uint8_t>(rows * (hidden / 16));
        plan->xq_pp = c.take<std::uint8_t>(plan->pp_rows * (hidden / 2));
        plan->xs_sw = c.take<std::uint8_t>(plan->pp_rows * (hidden / 16));
        plan->hq_pp = c.take<std::uint8_t>(plan->pp_rows * (intermediate / 2));
        plan->hs_sw = c.take<std::uint8_t>(plan->pp_rows * (intermediate / 16));
        plan->mixed_pp = c.take<std::uint16_t>(plan->pp_rows * hidden);
        plan->xq_tok = c.take<std::uint8_t>(static_cast<std::size_t>(16) * (hidden / 2));
        plan->xs_tok = c.take<std::uint8_t>(static_cast<std::size_t>(hidden / 64) * 512);
        plan->mega_sync = c.take<unsigned>(4);
        plan->gu_done = c.take<std::int32_t>(2 * 264);
        plan->ep_gu_done = c.take<std::int32_t>(2 * 264);
        plan->ep_logits = c.take<unsigned long long>(static_cast<std::size_t>(8) * kExperts);
        plan->mega_logits = c.take<unsigned long long>(static_cast<std::size_t>(16) * kExperts);
        plan->mega_ret = c.take<unsigned long long>(static_cast<std::size_t>(16) * (kTop + 1) * 1280);
        plan->mega_trace = c.take<unsigned long long>(static_cast<std::size_t>(plan->sm_count) * 64);
        plan->w_norms = c.take<float>(2 * kExperts);
        plan->router_stats = c.take<int>(2);
        plan->logit_partials = c.take<float>(static_cast<std::size_t>(kRouterSplits) * std::min(max_rows, kRouterSplitRows) * kExperts);
        plan->mega_hidden = c.take<unsigned long long>(static_cast<std::size_t>(16) * (hidden / 2));
        plan->normed = c.take<std::uint16_t>(rows * hidden);
        plan->ep_words = 16 * (kExperts + 1);
        plan->ep_src_base = c.take<std::int32_t>(plan->ep_words);
        plan->ep_src_start = c.take<std::int32_t>(plan->ep_words);
        plan->ep_zero_counts = c.take<std::int32_t>(kExperts + 1);
        plan->epg_counts = c.take<std::int32_t>(kExperts + 1);
        plan->epg_offsets = c.take<std::int32_t>(kExperts + 2);
        plan->stage_in = c.take<std::uint16_t>(rows * hidden);
        plan->stage_out = c.take<std::uint16_t>(rows * hidden);
        plan->stage_in_b = c.take<std::uint16_t>(rows * hidden);
        plan->stage_out_b = c.take<std::uint16_t>(rows * hidden);
        plan->status = c.take<std::int32_t>(1);
        if (pass == 0) {
            plan->bytes = c.used;
            st = cudaMalloc(&plan->storage, plan->bytes);
            if (st != cudaSuccess) {
                delete plan;
                return cudaErrorMemoryAllocation;
            }
            st = cudaMemset(plan->storage, 0, plan->bytes);
            if (st != cudaSuccess) {
                cudaFree(plan->storage);
                delete plan;
                return st;
            }
        }
    }
    {
        static const int kBoxRows[4] = {16, 32, 64, 128};
        bool ok = true;
        for (int i = 0; i < 4; ++i) {
            ok = ok && make_operand_map(&plan->map_x[i], plan->xq_pp, plan->pp_rows, hidden / 2, kBoxRows[i]) == cudaSuccess;
            ok = ok && make_operand_map(&plan->map_h[i], plan->hq_pp, plan->pp_rows, intermediate / 2, kBoxRows[i]) ==
                           cudaSuccess;
        }
        ok = ok && make_operand_map(&plan->map_x_tok, plan->xq_tok, 16, hidden / 2, 16) == cudaSuccess;
        plan->tc_ready = ok;
    }
    *out = plan;
    return cudaSuccess;
}

int p92b_plan_set_path(p92b_plan* plan, int path) {
    if (plan == nullptr || (path != 0 && path != 2 && path != 3)) return cudaErrorInvalidValue;
    if (!plan->tc_ready) return cudaErrorNotSupported;
    plan->path = path;
    return cudaSuccess;
}

void p92b_plan_destroy(p92b_plan* plan) {
    if (plan == nullptr) return;
    for (cudaEvent_t& ev : plan->stage_events) {
        if (ev != nullptr) cudaEventDestroy(ev);
    }
    for (int i = 0; i < 2; ++i) {
        if (plan->in_ready[i] != nullptr) cudaEventDestroy(plan->in_ready[i]);
        if (plan->block_done[i] != nullptr) cudaEventDestroy(plan->block_done[i]);
        if (plan->out_done[i] != nullptr) cudaEventDestroy(plan->out_done[i]);
    }
    if (plan->copy_in_stream != nullptr) cudaStreamDestroy(plan->copy_in_stream);
    if (plan->copy_out_stream != nullptr) cudaStreamDestroy(plan->copy_out_stream);
    if (plan->storage != nullptr) cudaFree(plan->storage);
    delete plan;
}

size_t p92b_plan_bytes(const p92b_plan* plan) { return plan == nullptr ? 0 : plan->bytes; }

int p92b_plan_stage_timing(p92b_plan* plan, int enable) {
    if (plan == nullptr) return cudaErrorInvalidValue;
    if (enable) {
        for (cudaEvent_t& ev : plan->stage_events) {
            if (ev == nullptr) {
                cudaError_t st = cudaEventCreate(&ev);
                if (st != cudaSuccess) return st;
            }
        }
        for (float& ms : plan->stage_ms) ms = 0.0F;
        plan->timed_calls = 0;
    }
    plan->timing = enable != 0;
    return cudaSuccess;
}

int p92b_plan_stage_times(const p92b_plan* plan, float* host_ms, int* host_calls) {
    if (plan == nullptr || host_ms == nullptr || host_calls == nullptr) return cudaErrorInvalidValue;
    for (int i = 0; i < P92B_STAGES; ++i) host_ms[i] = plan->stage_ms[i];
    *host_calls = plan->timed_calls;
    return cudaSuccess;
}

int p92b_plan_last_launches(const p92b_plan* plan) { return plan == nullptr ? 0 : plan->last_launches; }

int p92b_plan_get_views(const p92b_plan* plan, p92b_plan_views* v) {
    if (plan == nullptr || v == nullptr) return cudaErrorInvalidValue;
    v->logits = plan->logits;
    v->expert_ids = plan->ids;
    v->expert_weights = plan->route_weights;
    v->order = plan->order;
    v->position = plan->position;
    v->counts = plan->counts;
    v->offsets = plan->offsets;
    v->mixed = plan->mixed_pp;
    v->mixed_index = plan->pp_of_flat;
    v->status = plan->status;
    v->router_stats = plan->router_stats;
    v->trace = plan->mega_trace;
    v->trace_blocks = plan->sm_count;
    return cudaSuccess;
}

int p92b_bf16_gemv_f32(const uint16_t* input, const uint16_t* weight, float* output, int rows, int columns,
                       void* stream) {
    return launch_router_logits(input, weight, output, 1, rows, columns, true, static_cast<cudaStream_t>(stream));
}

int p92b_bf16_gemm_f32(const uint16_t* input, const uint16_t* weight, float* output, int batch_rows, int rows,
                       int columns, void* stream) {
    return launch_router_logits(input, weight, output, batch_rows, rows, columns, false,
                                static_cast<cudaStream_t>(stream));
}

int p92b_router_top8_rows(const float* logits, const float* correction_bias, int32_t* expert_ids,
                          float* expert_weights, int rows, float routed_scale, void* stream) {
    return launch_router_top8(logits, correction_bias, expert_ids, expert_weights, rows, routed_scale,
                              static_cast<cudaStream_t>(stream));
}

int p92b_router_top8(const float* logits, const float* correction_bias, int32_t* expert_ids,
                     float* expert_weights, float routed_scale, void* stream) {
    return p92b_router_top8_rows(logits, correction_bias, expert_ids, expert_weights, 1, routed_scale, stream);
}

int p92b_moe_permute(p92b_plan* plan, const int32_t* expert_ids, int assignments, int32_t* order,
                     int32_t* position, int32_t* counts, int32_t* offsets, void* stream) {
    if (plan == nullptr) return cudaErrorInvalidValue;
    return launch_permute(plan, expert_ids, assignments, order, position, counts, offsets, false, 0, 0,
                          static_cast<cudaStream_t>(stream));
}

int p92b_moe_forward(p92b_plan* plan, const p92b_bank* bank, const uint16_t* input,
                     const uint16_t* router_weight, const float* correction_bias, uint16_t* output, int rows,
                     float routed_scale, void* stream_) {
    return p92b_moe_forward_normed(plan, bank, input, nullptr, nullptr, 0.0F, router_weight, correction_bias, output, rows,
                                   routed_scale, stream_);
}

int p92b_moe_forward_normed(p92b_plan* plan, const p92b_bank* bank, const uint16_t* input, const uint16_t* pre_norm_weight,
                            const uint16_t* post_norm_weight, float norm_epsilon, const uint16_t* router_weight,
                            const float* correction_bias, uint16_t* output, int rows, float routed_scale, void* stream_) {
    if ((pre_norm_weight != nullptr || post_norm_weight != nullptr) && !(norm_epsilon > 0.0F)) return cudaErrorInvalidValue;
    if (plan == nullptr || bank == nullptr || input == nullptr || router_weight == nullptr ||
        correction_bias == nullptr || output == nullptr || rows <= 0 || rows > plan->max_rows ||
        !shapes_match(plan, bank) || bank->view.first_expert != 0 || bank->view.local_experts != kExperts) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int hidden = plan->hidden;
    plan->last_launches = 0;
    int stage = 0;
    // P92B_DEBUG_SYNC=1: synchronise after every stage so an asynchronous fault is reported by the
    // stage that caused it (printed to stderr); a debugging aid, never on in measurements
    static const bool debug_sync = std::getenv("P92B_DEBUG_SYNC") != nullptr;
    auto mark = [&]() -> cudaError_t {
        if (debug_sync) {
            const cudaError_t sync = cudaStreamSynchronize(stream);
            if (sync != cudaSuccess) {
                std::fprintf(stderr, "p92b_moe_forward: stage before mark %d failed: %s\n", stage, cudaGetErrorString(sync));
                return sync;
            }
        }
        if (!plan->timing) { ++stage; return cudaSuccess; }
        return cudaEventRecord(plan->stage_events[stage++], stream);
    };
    // programmatic dependent launch: each kernel's prologue (and, for the down kernel, its weight
    // prefetch) overlaps the tail of the one before; P92B_NO_PDL=1 switches it off for A/B timing
    static const bool pdl = std::getenv("P92B_NO_PDL") == nullptr;
    if (!plan->tc_ready || !bank->tc_ready) return cudaErrorNotSupported;
    // the single-kernel form is written for the model's expert shape; other shapes take the multi-kernel pipeline
    const bool mega_shape = plan->hidden == 2560 && plan->intermediate == 1024;
    if (plan->path == 3 && (rows > decode_mega_max_rows() || !mega_shape)) return cudaErrorInvalidValue;
    plan->last_path = 2;
    if (plan->path != 2 && rows <= decode_mega_max_rows() && mega_shape) {
        // the whole block as one persistent kernel; in timing mode its time is reported as stage 0
        cudaError_t st = mark();
        if (st != cudaSuccess) return st;
        st = launch_decode_mega(plan, bank, input, router_weight, correction_bias, output, rows, routed_scale, stream,
                                pdl, pre_norm_weight, post_norm_weight, norm_epsilon);
        if (st != cudaSuccess) return st;
        for (int i = 0; i < P92B_STAGES; ++i) {
            if ((st = mark()) != cudaSuccess) return st;
        }
        if (plan->timing) {
            if ((st = cudaStreamSynchronize(stream)) != cudaSuccess) return st;
            for (int i = 0; i < P92B_STAGES; ++i) {
                float ms = 0.0F;
                if ((st = cudaEventElapsedTime(&ms, plan->stage_events[i], plan->stage_events[i + 1])) != cudaSuccess) return st;
                plan->stage_ms[i] += ms;
            }
            plan->timed_calls += 1;
        }
        return cudaSuccess;
    }
    const int pad_align = tc_pad_align(rows);
    const int tile_rows = tc_tile_rows(rows);
    cudaError_t st = cudaSuccess;
    if (pre_norm_weight != nullptr) {
        // the multi-kernel pipeline reads the token rows in three kernels: normalise them once into the plan's scratch
        st = launch_rmsnorm(input, pre_norm_weight, plan->normed, rows, hidden, hidden, hidden, norm_epsilon, stream, pdl);
        if (st != cudaSuccess) return st;
        input = plan->normed;
        plan->last_launches += 1;
    }
    if ((st = mark()) != cudaSuccess) return st;
    // large batches: tensor-core logits with exact repair of the candidates (ids and weights still the reference's bit
    // for bit); in the stage table its three kernels are the "router logits" stage and the top-8 stage is empty
    bool routed = false;
    if (rows >= router_fast_min_rows()) {
        st = launch_router_fast(plan, input, router_weight, correction_bias, rows, routed_scale, stream, pdl);
        if (st == cudaSuccess) routed = true;
        else if (st != cudaErrorNotSupported) return st;
    }
    if (!routed) {
        st = launch_router_logits(input, router_weight, plan->logits, rows, kExperts, hidden, rows == 1, stream, pdl);
        if (st != cudaSuccess) return st;
        plan->last_launches += 1;
    }
    if ((st = mark()) != cudaSuccess) return st;
    if (rows <= route_fused_max_rows()) {
        // top-8, permutation and token quantisation as one block (stages 1-3 of the timing table)
        st = launch_route_fused(plan, correction_bias, routed_scale, input, rows, pad_align, tile_rows, stream, pdl);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
    } else {
        if (!routed) {
            st = launch_router_top8(plan->logits, correction_bias, plan->ids, plan->route_weights, rows, routed_scale, stream,
                                    pdl);
            if (st != cudaSuccess) return st;
            plan->last_launches += 1;
        }
        if ((st = mark()) != cudaSuccess) return st;
        st = launch_permute(plan, plan->ids, rows * kTop, plan->order, plan->position, plan->counts, plan->offsets, true,
                            pad_align, tile_rows, stream, pdl);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        st = launch_quantize_padded(plan, input, rows, stream, pdl);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        plan->last_launches += 1;
    }
    st = launch_experts_tc(plan, bank, rows, false, stream, pdl);
    if (st != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    st = launch_experts_tc(plan, bank, rows, true, stream, pdl);
    if (st != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    st = launch_combine_shared(plan->mixed_pp, plan->pp_of_flat, plan->route_weights, output, rows, hidden, stream, pdl);
    plan->last_launches += 3;
    if (st != cudaSuccess) return st;
    if (post_norm_weight != nullptr) {
        // in place: a block holds its whole row in shared memory before it writes
        st = launch_rmsnorm(output, post_norm_weight, output, rows, hidden, hidden, hidden, norm_epsilon, stream, pdl);
        if (st != cudaSuccess) return st;
        plan->last_launches += 1;
    }
    if (debug_sync && !plan->timing && (st = mark()) != cudaSuccess) return st;
    if (plan->timing) {
        if ((st = mark()) != cudaSuccess) return st;
        if ((st = cudaStreamSynchronize(stream)) != cudaSuccess) return st;
        for (int i = 0; i < P92B_STAGES; ++i) {
            float ms = 0.0F;
            if ((st = cudaEventElapsedTime(&ms, plan->stage_events[i], plan->stage_events[i + 1])) != cudaSuccess) return st;
            plan->stage_ms[i] += ms;
        }
        plan->timed_calls += 1;
    }
    return cudaSuccess;
}

int p92b_dense_forward(p92b_plan* plan, const p92b_bank* bank, const uint16_t* input, uint16_t* output, int rows,
                       void* stream_) {
    if (plan == nullptr || bank == nullptr || input == nullptr || output == nullptr || rows <= 0 || rows > plan->max_rows ||
        !shapes_match(plan, bank)) {
        return cudaErrorInvalidValue;
    }
    if (!plan->tc_ready || !bank->tc_ready) return cudaErrorNotSupported;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    static const bool pdl = std::getenv("P92B_NO_PDL") == nullptr;
    plan->last_launches = 0;
    plan->last_path = 2;
    // the MLP is the bank's last entry; every row is "routed" to it and to nothing else, so its rows sit at padded
    // positions 0 .. rows-1 in token order and the down product can write the caller's rows directly
    cudaError_t st = launch_dense_lists(plan, rows, tc_tile_rows(rows), stream, pdl);
    if (st != cudaSuccess) return st;
    st = launch_quantize_rows_to_pp(input, nullptr, plan->xq_pp, plan->xs_sw, rows, plan->hidden, stream, pdl);
    if (st != cudaSuccess) return st;
    st = launch_experts_tc(plan, bank, rows, false, stream, pdl);
    if (st != cudaSuccess) return st;
    TcIo io {};
    io.down_out = output;
    st = launch_experts_tc(plan, bank, rows, true, stream, pdl, &io);
    plan->last_launches += 3;
    return st;
}

int p92b_moe_forward_host(p92b_plan* plan, const p92b_bank* bank, const uint16_t* host_input,
                          const uint16_t* router_weight, const float* correction_bias, uint16_t* host_output,
                          int rows, float routed_scale, void* stream_) {
    if (plan == nullptr || host_input == nullptr || host_output == nullptr || rows <= 0 || rows > plan->max_rows) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const std::size_t bytes = static_cast<std::size_t>(rows) * plan->hidden * sizeof(std::uint16_t);
    cudaError_t st = cudaMemcpyAsync(plan->stage_in, host_input, bytes, cudaMemcpyHostToDevice, stream);
    if (st != cudaSuccess) return st;
    st = static_cast<cudaError_t>(p92b_moe_forward(plan, bank, plan->stage_in, router_weight, correction_bias,
                                                   plan->stage_out, rows, routed_scale, stream_));
    if (st != cudaSuccess) return st;
    st = cudaMemcpyAsync(host_output, plan->stage_out, bytes, cudaMemcpyDeviceToHost, stream);
    if (st != cudaSuccess) return st;
    return cudaStreamSynchronize(stream);
}

// Pipelined host calls.  Three streams: the caller's (the block), one for rows coming in, one for rows
// going out; two sets of staging rows used alternately.  Call n (set b = n & 1):
//   in stream    waits until block n-2 has read set b, copies the rows in, records in_ready[b]
//   caller's     waits for in_ready[b] and for the copy-out of call n-2 (it read set b), runs the block,
//                records block_done[b]
//   out stream   waits for block_done[b], copies the rows out, records out_done[b]
// so the copies of a call overlap the blocks of its neighbours, and the caller's stream never carries a copy.
static cudaError_t host_pipeline_setup(p92b_plan* plan) {
    if (plan->copy_in_stream != nullptr) return cudaSuccess;
    cudaError_t st = cudaStreamCreateWithFlags(&plan->copy_in_stream, cudaStreamNonBlocking);
    if (st == cudaSuccess) st = cudaStreamCreateWithFlags(&plan->copy_out_stream, cudaStreamNonBlocking);
    for (int i = 0; i < 2 && st == cudaSuccess; ++i) {
        st = cudaEventCreateWithFlags(&plan->in_ready[i], cudaEventDisableTiming);
        if (st == cudaSuccess) st = cudaEventCreateWithFlags(&plan->block_done[i], cudaEventDisableTiming);
        if (st == cudaSuccess) st = cudaEventCreateWithFlags(&plan->out_done[i], cudaEventDisableTiming);
    }
    return st;
}

}  // extern "C"

namespace p92b {

cudaError_t host_pipeline_begin(p92b_plan* plan, const std::uint16_t* pinned_input, int rows, cudaStream_t stream,
                                std::uint16_t** rows_in, std::uint16_t** rows_out, int* set) {
    cudaError_t st = host_pipeline_setup(plan);
    if (st != cudaSuccess) return st;
    const std::size_t bytes = static_cast<std::size_t>(rows) * plan->hidden * sizeof(std::uint16_t);
    const unsigned n = plan->host_calls++;
    const int b = static_cast<int>(n & 1U);
    *set = b;
    *rows_in = b == 0 ? plan->stage_in : plan->stage_in_b;
    *rows_out = b == 0 ? plan->stage_out : plan->stage_out_b;
    if (n >= 2 && (st = cudaStreamWaitEvent(plan->copy_in_stream, plan->block_done[b], 0)) != cudaSuccess) return st;
    if ((st = cudaMemcpyAsync(*rows_in, pinned_input, bytes, cudaMemcpyHostToDevice, plan->copy_in_stream)) != cudaSuccess) return st;
    if ((st = cudaEventRecord(plan->in_ready[b], plan->copy_in_stream)) != cudaSuccess) return st;
    if ((st = cudaStreamWaitEvent(stream, plan->in_ready[b], 0)) != cudaSuccess) return st;
    if (n >= 2 && (st = cudaStreamWaitEvent(stream, plan->out_done[b], 0)) != cudaSuccess) return st;
    return cudaSuccess;
}

cudaError_t host_pipeline_end(p92b_plan* plan, std::uint16_t* pinned_output, int rows, cudaStream_t stream, int set) {
    const std::size_t bytes = static_cast<std::size_t>(rows) * plan->hidden * sizeof(std::uint16_t);
    const std::uint16_t* rows_out = set == 0 ? plan->stage_out : plan->stage_out_b;
    cudaError_t st = cudaEventRecord(plan->block_done[set], stream);
    if (st != cudaSuccess) return st;
    if ((st = cudaStreamWaitEvent(plan->copy_out_stream, plan->block_done[set], 0)) != cudaSuccess) return st;
    if ((st = cudaMemcpyAsync(pinned_output, rows_out, bytes, cudaMemcpyDeviceToHost, plan->copy_out_stream)) != cudaSuccess) return st;
    return cudaEventRecord(plan->out_done[set], plan->copy_out_stream);
}

}  // namespace p92b

extern "C" {

int p92b_moe_forward_host_async(p92b_plan* plan, const p92b_bank* bank, const uint16_t* pinned_input,
                                const uint16_t* router_weight, const float* correction_bias, uint16_t* pinned_output,
                                int rows, float routed_scale, void* stream_) {
    if (plan == nullptr || pinned_input == nullptr || pinned_output == nullptr || rows <= 0 || rows > plan->max_rows) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    std::uint16_t *rows_in = nullptr, *rows_out = nullptr;
    int set = 0;
    cudaError_t st = host_pipeline_begin(plan, pinned_input, rows, stream, &rows_in, &rows_out, &set);
    if (st != cudaSuccess) return st;
    st = static_cast<cudaError_t>(p92b_moe_forward(plan, bank, rows_in, router_weight, correction_bias, rows_out, rows,
                                                   routed_scale, stream_));
    if (st != cudaSuccess) return st;
    return host_pipeline_end(plan, pinned_output, rows, stream, set);
}

int p92b_plan_host_flush(p92b_plan* plan, void* stream_) {
    if (plan == nullptr) return cudaErrorInvalidValue;
    if (plan->copy_out_stream == nullptr || plan->host_calls == 0) return cudaSuccess;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    cudaError_t st = cudaStreamWaitEvent(stream, plan->out_done[0], 0);
    if (st == cudaSuccess && plan->host_calls >= 2) st = cudaStreamWaitEvent(stream, plan->out_done[1], 0);
    return st;
}

int p92b_project_expert_gate_up(p92b_plan* plan, const p92b_bank* bank, const int32_t* expert_ids,
                                const uint16_t* input, uint16_t* gate_output, uint16_t* up_output, int rows,
                                void* stream_) {
    if (plan == nullptr || bank == nullptr || expert_ids == nullptr || input == nullptr || gate_output == nullptr ||
        up_output == nullptr || rows <= 0 || rows > plan->max_rows || !shapes_match(plan, bank)) {
        return cudaErrorInvalidValue;
    }
    if (!plan->tc_ready || !bank->tc_ready) return cudaErrorNotSupported;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    static const bool pdl = std::getenv("P92B_NO_PDL") == nullptr;
    plan->last_launches = 0;
    plan->last_path = 2;
    // permutation of the caller's ids -> token rows quantised into the padded position space -> the grouped
    // tcgen05 product with the epilogue that stores gate and up un-fused at their (row, slot) rows
    cudaError_t st = launch_permute(plan, expert_ids, rows * kTop, plan->order, plan->position, plan->counts,
                                    plan->offsets, true, tc_pad_align(rows), tc_tile_rows(rows), stream);
    if (st != cudaSuccess) return st;
    st = launch_quantize_padded(plan, input, rows, stream, pdl);
    if (st != cudaSuccess) return st;
    TcIo io {};
    io.gate_out = gate_output;
    io.up_out = up_output;
    io.out_row = plan->order;
    io.skip_shared = true;
    st = launch_experts_tc(plan, bank, rows, false, stream, pdl, &io);
    plan->last_launches += 2;
    return st;
}

int p92b_project_expert_down(p92b_plan* plan, const p92b_bank* bank, const int32_t* expert_ids,
                             const uint16_t* input_rows, uint16_t* output_rows, int rows, void* stream_) {
    if (plan == nullptr || bank == nullptr || expert_ids == nullptr || input_rows == nullptr ||
        output_rows == nullptr || rows <= 0 || rows > plan->max_rows || !shapes_match(plan, bank)) {
        return cudaErrorInvalidValue;
    }
    if (!plan->tc_ready || !bank->tc_ready) return cudaErrorNotSupported;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    static const bool pdl = std::getenv("P92B_NO_PDL") == nullptr;
    plan->last_launches = 0;
    plan->last_path = 2;
    cudaError_t st = launch_permute(plan, expert_ids, rows * kTop, plan->order, plan->position, plan->counts,
                                    plan->offsets, true, tc_pad_align(rows), tc_tile_rows(rows), stream);
    if (st != cudaSuccess) return st;
    // every (row, slot) intermediate row is quantised on its own (src/executor.cpp:85-91), to its padded position
    st = launch_quantize_rows_to_pp(input_rows, plan->pp_of_flat, plan->hq_pp, plan->hs_sw, rows * kTop, plan->intermediate,
                                    stream, pdl);
    if (st != cudaSuccess) return st;
    TcIo io {};
    io.down_out = output_rows;
    io.out_row = plan->order;
    io.skip_shared = true;
    io.wait_upstream = true;
    st = launch_experts_tc(plan, bank, rows, true, stream, pdl, &io);
    plan->last_launches += 2;
    return st;
}

// ---- stand-ins for the reference's grouped-projection plan and call (include/p92/kernels.h:25-53) ------------------

struct p92b_grouped_plan {
    p92b_plan* inner = nullptr;
    int groups = 0, rows = 0, columns = 0;
};

int p92b_nvfp4_grouped_plan_create(p92b_grouped_plan** out, int groups, int rows, int columns) {
    if (out == nullptr) return cudaErrorInvalidValue;
    *out = nullptr;
    // the reference's checks (cuda/nvfp4_grouped.cu:227-230) plus what the tile stream needs
    if (groups <= 0 || groups % kTop != 0 || rows <= 0 || columns <= 0 || rows % 128 != 0 || columns % 256 != 0) {
        return cudaErrorInvalidValue;
    }
    p92b_grouped_plan* g = new (std::nothrow) p92b_grouped_plan();
    if (g == nullptr) return cudaErrorMemoryAllocation;
    g->groups = groups;
    g->rows = rows;
    g->columns = columns;
    // a gate/up plan (rows < columns: [intermediate x hidden]) keeps its operand rows on the hidden side of the
    // scratch, a down plan ([hidden x intermediate]) on the intermediate side
    const bool token_side = rows < columns;
    const int st = p92b_plan_create(&g->inner, groups / kTop, token_side ? columns : rows, token_side ? rows : columns);
    if (st != cudaSuccess) {
        delete g;
        return st;
    }
    *out = g;
    return cudaSuccess;
}

void p92b_nvfp4_grouped_plan_destroy(p92b_grouped_plan* plan) {
    if (plan == nullptr) return;
    p92b_plan_destroy(plan->inner);
    delete plan;
}

int p92b_nvfp4_grouped_plan_status(const p92b_grouped_plan* plan, const int32_t** device_status) {
    if (plan == nullptr || device_status == nullptr) return cudaErrorInvalidValue;
    *device_status = plan->inner->status;
    return cudaSuccess;
}

int p92b_nvfp4_grouped_rows(p92b_grouped_plan* plan, const uint8_t* packed_input, const uint8_t* input_scales_swizzled,
                            const p92b_expert_projection* expert_bank, const int32_t* expert_ids, uint16_t* first_output,
                            uint16_t* second_output, int projection_kind, int batch_rows, int expert_distinct_input_rows,
                            void* stream_) {
    // cuda/nvfp4_grouped.cu:354-359
    if (plan == nullptr || packed_input == nullptr || input_scales_swizzled == nullptr || expert_bank == nullptr ||
        expert_ids == nullptr || first_output == nullptr || projection_kind < 0 || projection_kind > 2 || batch_rows <= 0 ||
        plan->groups != batch_rows * (second_output != nullptr ? 2 * kTop : kTop)) {
        return cudaErrorInvalidValue;
    }
    if (second_output != nullptr && projection_kind != 0) return cudaErrorNotSupported;   // two outputs = gate and up
    p92b_plan* p = plan->inner;
    const bool token_side = plan->rows < plan->columns;
    const bool down = !token_side;
    if ((projection_kind == 2) != down) return cudaErrorInvalidValue;     // the plan was created for the other matrix shape
    if (!p->tc_ready) return cudaErrorNotSupported;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    static const bool pdl = std::getenv("P92B_NO_PDL") == nullptr;
    p->last_launches = 0;
    p->last_path = 2;
    const int assignments = batch_rows * kTop;
    // the reference orders its problems by (kind, expert) with ties in the original order
    // (cuda/nvfp4_grouped.cu:117-132); the same stable order groups the rows per expert here
    cudaError_t st = launch_permute(p, expert_ids, assignments, p->order, p->position, p->counts, p->offsets, true,
                                    tc_pad_align(batch_rows), tc_tile_rows(batch_rows), stream);
    if (st != cudaSuccess) return st;
    st = launch_gather_quantized_rows(packed_input, input_scales_swizzled, p->pp_of_flat, down ? p->hq_pp : p->xq_pp,
                                      down ? p->hs_sw : p->xs_sw, assignments, plan->columns / 2,
                                      expert_distinct_input_rows != 0, stream, pdl);
    if (st != cudaSuccess) return st;
    TcIo io {};
    io.table = expert_bank;
    io.table_kind = projection_kind;
    io.out_row = p->order;
    io.skip_shared = true;
    if (second_output != nullptr) {
        io.gate_out = first_output;
        io.up_out = second_output;
    } else {
        io.down_out = first_output;
        io.single_matrix = !down;
    }
    st = launch_experts_tc(p, nullptr, batch_rows, down, stream, pdl, &io);
    p->last_launches += 2;
    return st;
}

int p92b_nvfp4_grouped_m1(p92b_grouped_plan* plan, const uint8_t* packed_input, const uint8_t* input_scales_swizzled,
                          const p92b_expert_projection* expert_bank, const int32_t* expert_ids, uint16_t* first_output,
                          uint16_t* second_output, int projection_kind, int distinct_input_rows, void* stream) {
    return p92b_nvfp4_grouped_rows(plan, packed_input, input_scales_swizzled, expert_bank, expert_ids, first_output,
                                   second_output, projection_kind, 1, distinct_input_rows, stream);
}

}  // extern "C"
