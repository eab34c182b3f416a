// Host-only parts of the C ABI: CSF block-scale codec, the schedules that feed the step
// scalars, whole-matrix sharding and the NCCL all-gather plumbing.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <new>
#include <numeric>
#include <vector>

#include "../../include/llmini_b200.h"

namespace {

// crates/cuda-kernels/src/utils/nvfp4/csf.rs:19-35
inline uint32_t code_offset(uint32_t r) { return (r / 16) * 96 + (r % 8) * 12 + (r % 16 / 8) * 3; }
inline uint32_t compact6(uint32_t w) {
    return (w & 63) | ((w & 0x3f00) >> 2) | ((w & 0x3f0000) >> 4) | ((w & 0x3f000000) >> 6);
}
inline uint8_t high1(uint32_t w) { return (uint8_t)((((w >> 6) & 0x01010101u) * 0x01020408u) >> 24); }
inline uint8_t high2(uint32_t w) {
    uint32_t v = (w >> 6) & 0x03030303u;
    v = (v | (v >> 6)) & 0x000f000fu;
    return (uint8_t)((v | (v >> 12)) & 255);
}
inline void put_u32(uint8_t *p, uint32_t v) { std::memcpy(p, &v, 4); }
inline uint32_t get_u32(const uint8_t *p) { uint32_t v; std::memcpy(&v, p, 4); return v; }

}  // namespace

extern "C" {

size_t b2_csf_encoded_len(size_t rows, size_t k) {
    if (rows == 1) return 128 + k / 16;
    return 128 + ((rows + 127) / 128) * ((k + 127) / 128) * 896;
}

size_t b2_csf_encode_host(const uint8_t *raw, size_t raw_len, size_t rows, size_t k, uint8_t *out,
                          size_t out_capacity) {
    if (!out || (!raw && raw_len)) return 0;
    if (k < 128 || k % 128 != 0 || rows == 0) return 0;
    if (rows * k > 0xffffffffull || raw_len > rows * k / 16) return 0;
    if (rows == 1) {  // csf.rs:180-189 (encode_vector)
        size_t n = 128 + k / 16;
        if (out_capacity < n) return 0;
        std::memset(out, 0, n);
        put_u32(out, (uint32_t)k);
        put_u32(out + 4, 1);
        out[8] = 255;
        out[9] = 8;
        if (raw_len) std::memcpy(out + 128, raw, raw_len);
        return n;
    }
    // csf.rs:51-95 (encode_matrix)
    int bytes = 1;
    for (size_t i = 0; i < raw_len; ++i)
        if (raw[i] >= 128) { bytes = 2; break; }
    const size_t stride = 768 + 128 * (size_t)bytes;
    const size_t padded = (rows + 127) / 128 * 128;
    const size_t n = 128 + padded / 128 * (k / 128) * stride;
    if (out_capacity < n) return 0;
    std::memset(out, 0, n);
    put_u32(out, (uint32_t)k);
    put_u32(out + 4, (uint32_t)rows);
    out[8] = (uint8_t)__builtin_ctzll(k / 16);
    out[9] = (uint8_t)(6 + bytes);
    const size_t groups = k / 16;
    for (size_t row = 0; row < rows; ++row) {
        for (size_t kg = 0; kg < groups; kg += 8) {
            uint8_t v[8];
            for (size_t i = 0; i < 8; ++i) {
                size_t idx = row * groups + kg + i;
                v[i] = idx < raw_len ? raw[idx] : 0;
            }
            uint32_t a = get_u32(v), b = get_u32(v + 4);
            size_t t = row / 128 * (k / 128) + kg / 8;
            size_t at = 128 + t * stride + code_offset((uint32_t)(row % 128));
            uint32_t ca = compact6(a), cb = compact6(b);
            out[at] = (uint8_t)ca; out[at + 1] = (uint8_t)(ca >> 8); out[at + 2] = (uint8_t)(ca >> 16);
            out[at + 6] = (uint8_t)cb; out[at + 7] = (uint8_t)(cb >> 8); out[at + 8] = (uint8_t)(cb >> 16);
            size_t am = 128 + t * stride + 768 + (row % 128) * (size_t)bytes;
            if (bytes == 1) out[am] = (uint8_t)(high1(a) | (high1(b) << 4));
            else { out[am] = high2(a); out[am + 1] = high2(b); }
        }
    }
    return n;
}

uint8_t b2_csf_scale_at(const uint8_t *s, size_t g) {
    if (s[8] == 255) return s[128 + g];  // csf.rs:190-192
    const uint32_t k = get_u32(s), groups = k / 16;
    const uint32_t row = (uint32_t)(g / groups), kg = (uint32_t)(g % groups);
    const uint32_t bytes = (uint32_t)s[9] - 6;
    const uint8_t *d = s + 128;
    const uint32_t t = row / 128 * (k / 128) + kg / 8, r = row % 128, stride = 768 + 128 * bytes;
    const size_t at = (size_t)t * stride + code_offset(r) + (kg % 8 / 4) * 6;
    const uint32_t shift = (kg % 4) * 6, bits = shift % 8;
    const size_t byte = at + shift / 8;
    const uint32_t lo = d[byte], hi = bits > 2 ? d[byte + 1] : 0;
    const uint8_t q = (uint8_t)(((lo | (hi << 8)) >> bits) & 63);
    const size_t am = (size_t)t * stride + 768 + (size_t)r * bytes;
    if (bytes == 1) return (uint8_t)(q | (((d[am] >> (kg % 8)) & 1) << 6));
    return (uint8_t)(q | (((d[am + kg % 8 / 4] >> ((kg % 4) * 2)) & 3) << 6));
}

float b2_warmup_multiplier(uint32_t step, uint32_t warmup_steps, float start_ratio) {
    if (step < 1) step = 1;
    if (step <= warmup_steps) {
        float progress = (float)step / (float)warmup_steps;
        return start_ratio + (1.0f - start_ratio) * progress;
    }
    return 1.0f;
}
float b2_schedule_free_beta(uint32_t step, uint32_t warmup_steps, float beta1, float rho) {
    if (step < 1) step = 1;
    uint32_t warmup = warmup_steps < 2 ? 2 : warmup_steps;
    if (step <= warmup) return beta1;
    float ratio = (float)(warmup - 1) / (float)(step - 1);
    return 1.0f - std::pow(ratio, rho) * (1.0f - beta1);
}
float b2_schedule_free_average_coefficient(uint32_t step, uint32_t warmup_steps, float start_ratio, float *weight_sum) {
    if (!weight_sum) return 0.0f;
    if (step < 1) step = 1;
    // AMUSE_AVERAGE_R = 0, AMUSE_WEIGHT_LR_POWER = 2 (src/training/learning_rate/schedule.rs:5-6)
    float lr_max = b2_warmup_multiplier(step, warmup_steps, start_ratio);
    float weight = std::pow((float)step, 0.0f) * std::pow(lr_max, 2.0f);
    *weight_sum += weight;
    return *weight_sum > 0.0f ? weight / *weight_sum : 0.0f;
}

int b2_shard_plan(const uint32_t *rows, const uint32_t *cols, uint32_t slot_count, uint32_t world, uint32_t *owner,
                  double *rank_flops) {
    if (!rows || !cols || !owner || world == 0) return B2_ERROR_INVALID_VALUE;
    std::vector<double> cost(slot_count), load(world, 0.0);
    std::vector<uint32_t> order(slot_count);
    std::iota(order.begin(), order.end(), 0u);
    for (uint32_t s = 0; s < slot_count; ++s) {
        double n = std::min(rows[s], cols[s]), m = std::max(rows[s], cols[s]);
        cost[s] = 4.0 * n * n * m + 2.0 * n * n * n;
    }
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return cost[a] > cost[b]; });
    for (uint32_t s : order) {
        uint32_t best = 0;
        for (uint32_t r = 1; r < world; ++r)
            if (load[r] < load[best]) best = r;
        owner[s] = best;
        load[best] += cost[s];
    }
    if (rank_flops) std::copy(load.begin(), load.end(), rank_flops);
    return B2_SUCCESS;
}

// ---- NCCL through the process's libnccl ------------------------------------------------------
struct nccl_uid { char internal[128]; };
struct nccl_api {
    void *handle = nullptr;
    int (*GetUniqueId)(nccl_uid *) = nullptr;
    int (*CommInitRank)(void **, int, nccl_uid, int) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    bool ok = false;
};
static nccl_api &nccl() {
    static nccl_api api;
    if (!api.handle) {
        api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) {
            api.GetUniqueId = reinterpret_cast<int (*)(nccl_uid *)>(dlsym(api.handle, "ncclGetUniqueId"));
            api.CommInitRank = reinterpret_cast<int (*)(void **, int, nccl_uid, int)>(dlsym(api.handle, "ncclCommInitRank"));
            api.CommDestroy = reinterpret_cast<int (*)(void *)>(dlsym(api.handle, "ncclCommDestroy"));
            api.AllGather = reinterpret_cast<int (*)(const void *, void *, size_t, int, void *, cudaStream_t)>(
                dlsym(api.handle, "ncclAllGather"));
            api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather;
        }
    }
    return api;
}
struct b2_comm {
    void *comm = nullptr;
    int rank = 0, world = 1;
};

int b2_comm_unique_id(uint8_t unique_id[128]) {
    if (!unique_id) return B2_ERROR_INVALID_VALUE;
    nccl_api &n = nccl();
    if (!n.ok) return B2_ERROR_NOT_SUPPORTED;
    nccl_uid id;
    if (n.GetUniqueId(&id) != 0) return 999;
    std::memcpy(unique_id, id.internal, 128);
    return B2_SUCCESS;
}
int b2_comm_create(b2_comm **comm, const uint8_t unique_id[128], int rank, int world) {
    if (!comm || !unique_id || world < 1 || rank < 0 || rank >= world) return B2_ERROR_INVALID_VALUE;
    nccl_api &n = nccl();
    if (!n.ok) return B2_ERROR_NOT_SUPPORTED;
    b2_comm *c = new (std::nothrow) b2_comm();
    if (!c) return 2;
    nccl_uid id;
    std::memcpy(id.internal, unique_id, 128);
    c->rank = rank;
    c->world = world;
    if (n.CommInitRank(&c->comm, world, id, rank) != 0) { delete c; return 999; }
    *comm = c;
    return B2_SUCCESS;
}
void b2_comm_destroy(b2_comm *comm) {
    if (!comm) return;
    if (comm->comm && nccl().ok) nccl().CommDestroy(comm->comm);
    delete comm;
}
int b2_allgather_nvfp4(b2_comm *comm, void *d_arena, size_t bytes_per_rank, void *stream) {
    if (!comm || !d_arena) return B2_ERROR_INVALID_VALUE;
    if (bytes_per_rank == 0) return B2_SUCCESS;
    nccl_api &n = nccl();
    if (!n.ok) return B2_ERROR_NOT_SUPPORTED;
    const uint8_t *send = static_cast<const uint8_t *>(d_arena) + (size_t)comm->rank * bytes_per_rank;
    // ncclInt8 == 0; in place: the send buffer is this rank's slice of the receive buffer
    int rc = n.AllGather(send, d_arena, bytes_per_rank, 0, comm->comm, reinterpret_cast<cudaStream_t>(stream));
    return rc == 0 ? B2_SUCCESS : 999;
}

}  // extern "C"
