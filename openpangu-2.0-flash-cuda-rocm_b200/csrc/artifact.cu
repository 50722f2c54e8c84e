// Reader of the engine's NVFP4 weight container ("P92FP41") and the loader that turns one layer of it into an
// expert bank.  Host code only; the device work is the bank's own retiling (p92b_bank_create).
//
// Container (include/p92/nvfp4_artifact.h:11-34, written by cuda/nvfp4_pack.cu:264-305): a directory with
//   manifest.bin          48-byte header {magic "P92FP41\0", version 1, record_bytes 128, tensor_count, reserved 0,
//                         weight_bytes, scale_bytes, source_payload_bytes}, then tensor_count records of 128 bytes
//                         {name[96], rows, columns, weight_offset, scale_offset, weight_scale_2, reserved 0},
//                         sorted by name;
//   weights.nvfp4         packed E2M1, rows x columns/2 bytes per tensor at weight_offset;
//   scales.e4m3           linear E4M3 scales, rows x columns/16 bytes per tensor at scale_offset;
//   scales.swizzled.e4m3  optional: the same scales already 128x4-tiled, same offsets and size (src/swizzle_main.cpp:68,
//                         used by src/resident.cpp:101-116 when present).
// The checks are the reference reader's (src/nvfp4_artifact.cpp:65-111); what it reports with an exception is
// reported here with cudaErrorInvalidValue (or cudaErrorFileNotFound) and a message kept per thread.
#include "p92b_common.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

namespace {

#pragma pack(push, 1)
struct ManifestHeader {
    char magic[8];
    std::uint32_t version;
    std::uint32_t record_bytes;
    std::uint32_t tensor_count;
    std::uint32_t reserved;
    std::uint64_t weight_bytes;
    std::uint64_t scale_bytes;
    std::uint64_t source_payload_bytes;
};
struct ManifestRecord {
    char name[96];
    std::uint32_t rows;
    std::uint32_t columns;
    std::uint64_t weight_offset;
    std::uint64_t scale_offset;
    float weight_scale_2;
    std::uint32_t reserved;
};
#pragma pack(pop)
static_assert(sizeof(ManifestHeader) == 48 && sizeof(ManifestRecord) == 128, "container layout");
static_assert(sizeof(ManifestRecord) == sizeof(p92b_artifact_record), "public record mirrors the container's");

struct Mapping {
    void* base = nullptr;
    std::size_t bytes = 0;
};

thread_local std::string g_error;

int fail(int code, const std::string& message) {
    g_error = message;
    return code;
}

int map_read_only(const std::string& path, Mapping* out) {
    const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) return fail(cudaErrorFileNotFound, "cannot open " + path);
    struct stat st {};
    if (::fstat(fd, &st) != 0 || st.st_size <= 0) {
        ::close(fd);
        return fail(cudaErrorInvalidValue, "empty or unreadable file " + path);
    }
    void* base = ::mmap(nullptr, static_cast<std::size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (base == MAP_FAILED) return fail(cudaErrorInvalidValue, "cannot map " + path);
    out->base = base;
    out->bytes = static_cast<std::size_t>(st.st_size);
    return cudaSuccess;
}

void unmap(Mapping* m) {
    if (m->base != nullptr) ::munmap(m->base, m->bytes);
    *m = {};
}

std::string record_name(const ManifestRecord& r) {
    return std::string(r.name, ::strnlen(r.name, sizeof(r.name)));
}

}  // namespace

struct p92b_artifact {
    Mapping manifest, weights, scales, swizzled;
    const ManifestHeader* header = nullptr;
    const ManifestRecord* records = nullptr;
};

namespace {

const ManifestRecord* find_record(const p92b_artifact* a, const std::string& key) {
    const ManifestRecord* begin = a->records;
    const ManifestRecord* end = a->records + a->header->tensor_count;
    const ManifestRecord* it = std::lower_bound(begin, end, key, [](const ManifestRecord& r, const std::string& wanted) {
        return record_name(r) < wanted;
    });
    return it != end && record_name(*it) == key ? it : nullptr;
}

}  // namespace

extern "C" {

const char* p92b_artifact_last_error(void) { return g_error.c_str(); }

void p92b_artifact_close(p92b_artifact* a) {
    if (a == nullptr) return;
    unmap(&a->manifest);
    unmap(&a->weights);
    unmap(&a->scales);
    unmap(&a->swizzled);
    delete a;
}

int p92b_artifact_open(p92b_artifact** out, const char* directory) {
    if (out == nullptr) return cudaErrorInvalidValue;
    *out = nullptr;
    if (directory == nullptr) return fail(cudaErrorInvalidValue, "no directory");
    p92b_artifact* a = new (std::nothrow) p92b_artifact();
    if (a == nullptr) return cudaErrorMemoryAllocation;
    const std::string dir(directory);
    int st = map_read_only(dir + "/manifest.bin", &a->manifest);
    if (st == cudaSuccess) st = map_read_only(dir + "/weights.nvfp4", &a->weights);
    if (st == cudaSuccess) st = map_read_only(dir + "/scales.e4m3", &a->scales);
    auto reject = [&](int code, const std::string& message) {
        p92b_artifact_close(a);
        return fail(code, message);
    };
    if (st != cudaSuccess) return reject(st, g_error);
    if (a->manifest.bytes < sizeof(ManifestHeader)) return reject(cudaErrorInvalidValue, "short NVFP4 manifest");
    a->header = static_cast<const ManifestHeader*>(a->manifest.base);
    static const char kMagic[8] = {'P', '9', '2', 'F', 'P', '4', '1', '\0'};
    const std::uint64_t expected = sizeof(ManifestHeader) + static_cast<std::uint64_t>(a->header->tensor_count) * sizeof(ManifestRecord);
    if (std::memcmp(a->header->magic, kMagic, sizeof(kMagic)) != 0 || a->header->version != 1 ||
        a->header->record_bytes != sizeof(ManifestRecord) || a->header->reserved != 0 || expected != a->manifest.bytes) {
        return reject(cudaErrorInvalidValue, "NVFP4 manifest contract mismatch");
    }
    if (a->header->weight_bytes != a->weights.bytes || a->header->scale_bytes != a->scales.bytes) {
        return reject(cudaErrorInvalidValue, "NVFP4 artifact file-size mismatch");
    }
    a->records = reinterpret_cast<const ManifestRecord*>(static_cast<const std::uint8_t*>(a->manifest.base) + sizeof(ManifestHeader));
    std::string previous;
    for (std::uint32_t i = 0; i < a->header->tensor_count; ++i) {
        const ManifestRecord& r = a->records[i];
        const std::string current = record_name(r);
        if (current.empty() || (i != 0 && previous >= current) || r.reserved != 0 || r.rows == 0 || r.columns == 0 ||
            r.rows % 128 != 0 || r.columns % 16 != 0 || !(r.weight_scale_2 > 0.0F)) {
            return reject(cudaErrorInvalidValue, "invalid NVFP4 record: " + current);
        }
        const std::uint64_t packed = static_cast<std::uint64_t>(r.rows) * r.columns / 2;
        const std::uint64_t scale = static_cast<std::uint64_t>(r.rows) * r.columns / 16;
        if (r.weight_offset > a->weights.bytes || packed > a->weights.bytes - r.weight_offset ||
            r.scale_offset > a->scales.bytes || scale > a->scales.bytes - r.scale_offset) {
            return reject(cudaErrorInvalidValue, "NVFP4 record lies outside artifact: " + current);
        }
        previous = current;
    }
    // the pre-tiled scale file is optional; when present it must have the linear file's size (src/resident.cpp:101-107)
    Mapping tiled;
    if (::access((dir + "/scales.swizzled.e4m3").c_str(), R_OK) == 0) {
        st = map_read_only(dir + "/scales.swizzled.e4m3", &tiled);
        if (st != cudaSuccess) return reject(st, g_error);
        if (tiled.bytes != a->scales.bytes) {
            unmap(&tiled);
            return reject(cudaErrorInvalidValue, "pre-swizzled scale file size mismatch");
        }
        a->swizzled = tiled;
    }
    *out = a;
    return cudaSuccess;
}

int p92b_artifact_tensor_count(const p92b_artifact* a) { return a == nullptr ? 0 : static_cast<int>(a->header->tensor_count); }

int p92b_artifact_has_swizzled_scales(const p92b_artifact* a) { return a != nullptr && a->swizzled.base != nullptr ? 1 : 0; }

int p92b_artifact_at(const p92b_artifact* a, int index, p92b_artifact_record* out) {
    if (a == nullptr || out == nullptr || index < 0 || index >= static_cast<int>(a->header->tensor_count)) {
        return fail(cudaErrorInvalidValue, "NVFP4 record index");
    }
    std::memcpy(out, &a->records[index], sizeof(*out));
    return cudaSuccess;
}

int p92b_artifact_find(const p92b_artifact* a, const char* name, p92b_artifact_record* out) {
    if (a == nullptr || name == nullptr || out == nullptr) return cudaErrorInvalidValue;
    const ManifestRecord* r = find_record(a, name);
    if (r == nullptr) return fail(cudaErrorInvalidValue, std::string("missing NVFP4 tensor: ") + name);
    std::memcpy(out, r, sizeof(*out));
    return cudaSuccess;
}

const uint8_t* p92b_artifact_weight(const p92b_artifact* a, const p92b_artifact_record* r) {
    return a == nullptr || r == nullptr ? nullptr : static_cast<const std::uint8_t*>(a->weights.base) + r->weight_offset;
}

const uint8_t* p92b_artifact_scales(const p92b_artifact* a, const p92b_artifact_record* r) {
    return a == nullptr || r == nullptr ? nullptr : static_cast<const std::uint8_t*>(a->scales.base) + r->scale_offset;
}

// Uploads the (entries x gate/up/down) tensors named by `prefixes` into a staging area in the reference's resident
// form (packed weights, 128x4-tiled scales, alpha) and hands them to p92b_bank_create, which retiles them into the
// library's stream; the staging area is freed again.  Scales come from scales.swizzled.e4m3 when the container has
// it, otherwise the linear scales are uploaded and tiled on the device (src/resident.cpp:101-139 does the same).
static int bank_from_prefixes(p92b_bank** out, const p92b_artifact* a, const std::vector<std::string>& prefixes,
                              int first_expert, int local_experts, void* stream_) {
    static const char* kKinds[3] = {".gate_proj.weight", ".up_proj.weight", ".down_proj.weight"};
    const int entries = static_cast<int>(prefixes.size());
    std::vector<const ManifestRecord*> recs(static_cast<std::size_t>(entries) * 3);
    for (int e = 0; e < entries; ++e) {
        for (int k = 0; k < 3; ++k) {
            const std::string name = prefixes[e] + kKinds[k];
            recs[e * 3 + k] = find_record(a, name);
            if (recs[e * 3 + k] == nullptr) return fail(cudaErrorInvalidValue, "missing NVFP4 tensor: " + name);
        }
    }
    const std::uint32_t inter = recs[0]->rows, hidden = recs[0]->columns;
    for (int e = 0; e < entries; ++e) {
        const ManifestRecord* const* r = &recs[e * 3];
        if (r[0]->rows != inter || r[0]->columns != hidden || r[1]->rows != inter || r[1]->columns != hidden ||
            r[2]->rows != hidden || r[2]->columns != inter) {
            return fail(cudaErrorInvalidValue, "expert shapes differ inside the layer: " + prefixes[e]);
        }
    }
    if (hidden % 256 != 0 || inter % 512 != 0) return fail(cudaErrorInvalidValue, "expert shape not supported by the tile stream");
    const std::size_t packed = static_cast<std::size_t>(inter) * hidden / 2;
    const std::size_t scale = static_cast<std::size_t>(inter) * hidden / 16;
    const std::size_t n = recs.size();
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    std::uint8_t *d_weights = nullptr, *d_scales = nullptr, *d_linear = nullptr;
    float* d_alpha = nullptr;
    std::vector<float> alphas(n);
    std::vector<p92b_expert_projection> table(n);
    cudaError_t st = cudaMalloc(&d_weights, n * packed);
    if (st == cudaSuccess) st = cudaMalloc(&d_scales, n * scale);
    if (st == cudaSuccess) st = cudaMalloc(&d_alpha, n * sizeof(float));
    const bool tiled = a->swizzled.base != nullptr;
    if (st == cudaSuccess && !tiled) st = cudaMalloc(&d_linear, scale);
    for (std::size_t i = 0; i < n && st == cudaSuccess; ++i) {
        const ManifestRecord& r = *recs[i];
        st = cudaMemcpyAsync(d_weights + i * packed, static_cast<const std::uint8_t*>(a->weights.base) + r.weight_offset, packed,
                             cudaMemcpyHostToDevice, stream);
        if (st != cudaSuccess) break;
        if (tiled) {
            st = cudaMemcpyAsync(d_scales + i * scale, static_cast<const std::uint8_t*>(a->swizzled.base) + r.scale_offset, scale,
                                 cudaMemcpyHostToDevice, stream);
        } else {
            st = cudaMemcpyAsync(d_linear, static_cast<const std::uint8_t*>(a->scales.base) + r.scale_offset, scale,
                                 cudaMemcpyHostToDevice, stream);
            if (st == cudaSuccess) {
                st = static_cast<cudaError_t>(p92b_nvfp4_swizzle_scales(d_linear, d_scales + i * scale, static_cast<int>(r.rows),
                                                                        static_cast<int>(r.columns / 16), stream_));
            }
        }
        alphas[i] = r.weight_scale_2;
        table[i] = {d_weights + i * packed, d_scales + i * scale, d_alpha + i};
    }
    if (st == cudaSuccess) st = cudaMemcpyAsync(d_alpha, alphas.data(), n * sizeof(float), cudaMemcpyHostToDevice, stream);
    if (st == cudaSuccess) {
        st = static_cast<cudaError_t>(p92b_bank_create(out, table.data(), first_expert, local_experts, static_cast<int>(hidden),
                                                       static_cast<int>(inter), 0, stream_));     // synchronises the stream
    }
    cudaFree(d_linear);
    cudaFree(d_alpha);
    cudaFree(d_scales);
    cudaFree(d_weights);
    if (st != cudaSuccess) return fail(st, std::string("loading the bank failed: ") + cudaGetErrorString(st));
    return cudaSuccess;
}

int p92b_bank_create_from_artifact(p92b_bank** bank, const p92b_artifact* artifact, int layer_index, int first_expert,
                                   int local_experts, void* stream) {
    if (bank == nullptr) return cudaErrorInvalidValue;
    *bank = nullptr;
    if (artifact == nullptr || layer_index < 0 || first_expert < 0 || local_experts <= 0 ||
        first_expert + local_experts > p92b::kExperts) {
        return fail(cudaErrorInvalidValue, "invalid layer or expert range");
    }
    // the names Model::Impl::bind_weights binds (src/model.cpp:667-681,724): routed experts, then the shared expert
    const std::string layer = "model.layers." + std::to_string(layer_index) + ".mlp.";
    std::vector<std::string> prefixes;
    for (int e = 0; e < local_experts; ++e) prefixes.push_back(layer + "experts." + std::to_string(first_expert + e));
    prefixes.push_back(layer + "shared_experts");
    return bank_from_prefixes(bank, artifact, prefixes, first_expert, local_experts, stream);
}

int p92b_dense_bank_create_from_artifact(p92b_bank** bank, const p92b_artifact* artifact, int layer_index, void* stream) {
    if (bank == nullptr) return cudaErrorInvalidValue;
    *bank = nullptr;
    if (artifact == nullptr || layer_index < 0) return fail(cudaErrorInvalidValue, "invalid layer");
    // the dense MLP of layers 0-1 is bound as "model.layers.<l>.mlp" (src/model.cpp:720)
    return bank_from_prefixes(bank, artifact, {"model.layers." + std::to_string(layer_index) + ".mlp"}, 0, 0, stream);
}

}  // extern "C"
