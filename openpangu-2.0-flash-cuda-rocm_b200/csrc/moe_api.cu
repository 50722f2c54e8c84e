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
    std::size_t g13, g2, w13, w2, sf13, sf2, alpha, total;
};

BankLayout bank_layout(int entries, int hidden, int inter, bool stream_copy) {
    BankLayout l {};
    Carver c;
    const std::size_t e = static_cast<std::size_t>(entries);
    l.g13 = c.used; c.take<std::uint8_t>(e * (inter / 128) * (hidden / 256) * kChunkBytes);
    l.g2 = c.used; c.take<std::uint8_t>(e * (hidden / 128) * (inter / 512) * kChunkBytes);
    if (stream_copy) {
        l.w13 = c.used; c.take<std::uint8_t>(e * 2 * inter * (hidden / 2));
        l.w2 = c.used; c.take<std::uint8_t>(e * hidden * (inter / 2));
        l.sf13 = c.used; c.take<std::uint8_t>(e * 2 * inter * (hidden / 16));
        l.sf2 = c.used; c.take<std::uint8_t>(e * hidden * (inter / 16));
    }
    l.alpha = c.used; c.take<float>(e * 3);
    l.total = c.used;
    return l;
}

RouteView route_view(const p92b_plan* plan) {
    RouteView r {};
    r.counts = plan->counts;
    r.offsets = plan->offsets;
    r.row_token = plan->row_token;
    r.active = plan->active;
    r.active_count = plan->active_count;
    return r;
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
        intermediate % 512 != 0 || (flags & ~P92B_BANK_STREAM_COPY) != 0) {
        return cudaErrorInvalidValue;
    }
    const int entries = local_experts + 1;
    for (int i = 0; i < entries * 3; ++i) {
        if (host_entries[i].weight == nullptr || host_entries[i].scales_swizzled == nullptr ||
            host_entries[i].alpha == nullptr) {
            return cudaErrorInvalidValue;
        }
    }
    const bool stream_copy = (flags & P92B_BANK_STREAM_COPY) != 0;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    p92b_bank* bank = new (std::nothrow) p92b_bank();
    if (bank == nullptr) return cudaErrorMemoryAllocation;
    const BankLayout l = bank_layout(entries, hidden, intermediate, stream_copy);
    cudaError_t st = cudaMalloc(&bank->storage, l.total);
    if (st != cudaSuccess) {
        delete bank;
        return cudaErrorMemoryAllocation;
    }
    bank->bytes = l.total;
    std::uint8_t* base = static_cast<std::uint8_t*>(bank->storage);
    std::uint8_t* g13 = base + l.g13;
    std::uint8_t* g2 = base + l.g2;
    std::uint8_t* w13 = stream_copy ? base + l.w13 : nullptr;
    std::uint8_t* w2 = stream_copy ? base + l.w2 : nullptr;
    std::uint8_t* sf13 = stream_copy ? base + l.sf13 : nullptr;
    std::uint8_t* sf2 = stream_copy ? base + l.sf2 : nullptr;
    float* alpha = reinterpret_cast<float*>(base + l.alpha);

    const std::size_t gu_bytes = static_cast<std::size_t>(intermediate) * (hidden / 2);
    const std::size_t dn_bytes = static_cast<std::size_t>(hidden) * (intermediate / 2);
    const std::size_t gu_sf = static_cast<std::size_t>(intermediate) * (hidden / 16);
    const std::size_t dn_sf = static_cast<std::size_t>(hidden) * (intermediate / 16);
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
    if (stream_copy) {
        for (int e = 0; e < entries; ++e) {
            for (int kind = 0; kind < 3; ++kind) {
                const p92b_expert_projection& src = host_entries[e * 3 + kind];
                if (kind < 2) {
                    BANK_TRY(cudaMemcpyAsync(w13 + (static_cast<std::size_t>(e) * 2 + kind) * gu_bytes, src.weight,
                                             gu_bytes, cudaMemcpyDeviceToDevice, stream));
                    BANK_TRY(launch_unswizzle(src.scales_swizzled,
                                              sf13 + (static_cast<std::size_t>(e) * 2 + kind) * gu_sf, intermediate,
                                              hidden / 16, stream));
                } else {
                    BANK_TRY(cudaMemcpyAsync(w2 + static_cast<std::size_t>(e) * dn_bytes, src.weight, dn_bytes,
                                             cudaMemcpyDeviceToDevice, stream));
                    BANK_TRY(launch_unswizzle(src.scales_swizzled, sf2 + static_cast<std::size_t>(e) * dn_sf, hidden,
                                              intermediate / 16, stream));
                }
            }
        }
    }
    BANK_TRY(cudaStreamSynchronize(stream));
#undef BANK_TRY
    cudaFree(device_table);
    bank->view.g13 = g13;
    bank->view.g2 = g2;
    bank->view.w13 = w13;
    bank->view.w2 = w2;
    bank->view.sf13 = sf13;
    bank->view.sf2 = sf2;
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
        plan->xq = c.take<std::uint8_t>(rows * (hidden / 2));
        plan->xs = c.take<std::uint8_t>(rows * (hidden / 16));
        plan->hq = c.take<std::uint8_t>(rows * (kTop + 1) * (intermediate / 2));
        plan->hs = c.take<std::uint8_t>(rows * (kTop + 1) * (intermediate / 16));
        plan->mixed = c.take<std::uint16_t>(rows * (kTop + 1) * hidden);
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
        plan->mega_logits = c.take<unsigned long long>(static_cast<std::size_t>(8) * kExperts);
        plan->mega_ret = c.take<unsigned long long>(static_cast<std::size_t>(8) * (kTop + 1) * 1280);
        plan->mega_trace = c.take<unsigned long long>(static_cast<std::size_t>(plan->sm_count) * 64);
        plan->mega_hidden = c.take<unsigned long long>(static_cast<std::size_t>(8) * (hidden / 2));
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
    if (plan == nullptr || path < 0 || path > 3) return cudaErrorInvalidValue;
    if (path >= 2 && !plan->tc_ready) return cudaErrorNotSupported;
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
    v->mixed = plan->last_path == 2 ? plan->mixed_pp : plan->mixed;
    v->mixed_index = plan->pp_of_flat;
    v->status = plan->status;
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
    const bool tc = plan->path >= 2 || (plan->path == 0 && plan->tc_ready && bank->tc_ready);
    if (tc && (!plan->tc_ready || !bank->tc_ready)) return cudaErrorNotSupported;
    // the single-kernel form is written for the model's expert shape; other shapes take the multi-kernel pipeline
    const bool mega_shape = plan->hidden == 2560 && plan->intermediate == 1024;
    if (plan->path == 3 && (rows > decode_mega_max_rows() || !mega_shape)) return cudaErrorInvalidValue;
    plan->last_path = tc ? 2 : 1;
    if (tc && plan->path != 2 && rows <= decode_mega_max_rows() && mega_shape) {
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
    const int pad_align = tc ? tc_pad_align(rows) : 1;
    const int tile_rows = tc ? tc_tile_rows(rows) : (1 << 30);
    cudaError_t st = cudaSuccess;
    if (pre_norm_weight != nullptr) {
        // the multi-kernel pipeline reads the token rows in three kernels: normalise them once into the plan's scratch
        st = launch_rmsnorm(input, pre_norm_weight, plan->normed, rows, hidden, hidden, hidden, norm_epsilon, stream, pdl);
        if (st != cudaSuccess) return st;
        input = plan->normed;
        plan->last_launches += 1;
    }
    if ((st = mark()) != cudaSuccess) return st;
    st = launch_router_logits(input, router_weight, plan->logits, rows, kExperts, hidden, rows == 1, stream, pdl);
    if (st != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    plan->last_launches += 1;
    if (tc && rows <= route_fused_max_rows()) {
        // top-8, permutation and token quantisation as one block (stages 1-3 of the timing table)
        st = launch_route_fused(plan, correction_bias, routed_scale, input, rows, pad_align, tile_rows, stream, pdl);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
    } else {
        st = launch_router_top8(plan->logits, correction_bias, plan->ids, plan->route_weights, rows, routed_scale, stream,
                                pdl);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        plan->last_launches += 1;
        st = launch_permute(plan, plan->ids, rows * kTop, plan->order, plan->position, plan->counts, plan->offsets, true,
                            pad_align, tile_rows, stream, pdl);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        if (tc) {
            st = launch_quantize_padded(plan, input, rows, stream, pdl);
        } else {
            st = launch_quantize(input, plan->xq, plan->xs, static_cast<long>(rows) * hidden / 16, 1.0F, stream);
        }
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        plan->last_launches += 1;
    }
    if (tc) {
        st = launch_experts_tc(plan, bank, rows, false, stream, pdl);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        st = launch_experts_tc(plan, bank, rows, true, stream, pdl);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        st = launch_combine_shared(plan->mixed_pp, plan->pp_of_flat, plan->route_weights, output, rows, hidden, stream,
                                   pdl);
    } else {
        const RouteView route = route_view(plan);
        st = launch_gate_up(plan, bank->view, route, plan->xq, plan->xs, plan->hq, plan->hs, nullptr, nullptr,
                            plan->order, rows, stream);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        st = launch_down(plan, bank->view, route, plan->hq, plan->hs, plan->mixed, nullptr, nullptr, 0, stream);
        if (st != cudaSuccess) return st;
        if ((st = mark()) != cudaSuccess) return st;
        st = launch_combine_shared(plan->mixed, plan->pp_of_flat, plan->route_weights, output, rows, hidden, stream);
    }
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
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    plan->last_launches = 0;
    cudaError_t st = launch_permute(plan, expert_ids, rows * kTop, plan->order, plan->position, plan->counts,
                                    plan->offsets, true, 1, 1 << 30, stream);
    if (st != cudaSuccess) return st;
    st = launch_quantize(input, plan->xq, plan->xs, static_cast<long>(rows) * plan->hidden / 16, 1.0F, stream);
    if (st != cudaSuccess) return st;
    st = launch_gate_up(plan, bank->view, route_view(plan), plan->xq, plan->xs, nullptr, nullptr, gate_output,
                        up_output, plan->order, rows, stream);
    plan->last_launches += 2;
    return st;
}

int p92b_project_expert_down(p92b_plan* plan, const p92b_bank* bank, const int32_t* expert_ids,
                             const uint16_t* input_rows, uint16_t* output_rows, int rows, void* stream_) {
    if (plan == nullptr || bank == nullptr || expert_ids == nullptr || input_rows == nullptr ||
        output_rows == nullptr || rows <= 0 || rows > plan->max_rows || !shapes_match(plan, bank)) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    plan->last_launches = 0;
    cudaError_t st = launch_permute(plan, expert_ids, rows * kTop, plan->order, plan->position, plan->counts,
                                    plan->offsets, true, 1, 1 << 30, stream);
    if (st != cudaSuccess) return st;
    // every (row, slot) intermediate row is quantised on its own (src/executor.cpp:85-91), in flat order
    st = launch_quantize(input_rows, plan->hq, plan->hs, static_cast<long>(rows) * kTop * plan->intermediate / 16, 1.0F,
                         stream);
    if (st != cudaSuccess) return st;
    st = launch_down(plan, bank->view, route_view(plan), plan->hq, plan->hs, output_rows, plan->order, plan->order, 1,
                     stream);
    plan->last_launches += 2;
    return st;
}

}  // extern "C"
