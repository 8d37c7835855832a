// Request dispatcher for the GPUs of one box (include/s1_dispatch.h): whole requests assigned to
// ranks by estimated cost, each rank's share prefilled in packs through the host executor, the
// decision logits gathered to rank 0 by one NCCL all-gather. NCCL is bound at run time.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <chrono>
#include <string>
#include <thread>
#include <vector>

#include "cs1_ops.h"
#include "s1_dispatch.h"
#include "s1_executor.h"

namespace {

#define D_TRY(expr)               \
    do {                          \
        const int rc_ = (expr);   \
        if (rc_ != 0) return rc_; \
    } while (0)

// The NCCL entry points this file uses, resolved from libnccl.so.2 on first need.
struct Nccl {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;

    int load(const char* path) {
        lib = dlopen(path && path[0] ? path : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!lib) return S1_ERR_DISPATCH_NCCL;
        auto sym = [&](const char* name) { return dlsym(lib, name); };
        GetUniqueId = reinterpret_cast<decltype(GetUniqueId)>(sym("ncclGetUniqueId"));
        CommInitRank = reinterpret_cast<decltype(CommInitRank)>(sym("ncclCommInitRank"));
        CommDestroy = reinterpret_cast<decltype(CommDestroy)>(sym("ncclCommDestroy"));
        AllGather = reinterpret_cast<decltype(AllGather)>(sym("ncclAllGather"));
        AllReduce = reinterpret_cast<decltype(AllReduce)>(sym("ncclAllReduce"));
        return GetUniqueId && CommInitRank && CommDestroy && AllGather && AllReduce ? 0 : S1_ERR_DISPATCH_NCCL;
    }
};

struct Dispatch {
    int rank = 0, world = 1, device = 0;
    Nccl nccl;
    ncclComm_t comm = nullptr;
    cudaStream_t side = nullptr;  // the harness collectives, which have no model
    double* side_dev = nullptr;   // their device staging
    size_t side_cap = 0;
    double a = 1.0, b = 4e-6;
    std::vector<double> speed;  // per rank, relative; empty = all equal

    // the plan
    void* model = nullptr;
    int hidden = 0, n_classes = 0, n = 0, most = 0;
    std::vector<int> lengths, rank_of;
    std::vector<std::vector<int>> members;  // per rank: its requests in run order
    std::vector<int> local_len, pack_start;
    std::vector<size_t> token_at;  // first token of each local request in the local id buffers
    size_t local_tokens = 0;
    bool staged = false, uploaded = false, queued = false;

    int32_t* ids_pinned = nullptr;
    int32_t* ids_device = nullptr;
    void* rows_device = nullptr;
    uint16_t* rows_host = nullptr;
    float *block_host = nullptr, *block_dev = nullptr, *all_dev = nullptr, *all_host = nullptr;
    std::vector<cudaEvent_t> pack_events;  // two per pack
};

int nccl_rc(ncclResult_t r) { return r == ncclSuccess ? 0 : S1_ERR_DISPATCH_COMM; }

void release_plan(Dispatch* d) {
    if (d->ids_pinned) cudaFreeHost(d->ids_pinned);
    if (d->ids_device) cudaFree(d->ids_device);
    if (d->rows_device) cudaFree(d->rows_device);
    if (d->rows_host) cudaFreeHost(d->rows_host);
    if (d->block_host) cudaFreeHost(d->block_host);
    if (d->block_dev) cudaFree(d->block_dev);
    if (d->all_dev) cudaFree(d->all_dev);
    if (d->all_host) cudaFreeHost(d->all_host);
    for (cudaEvent_t e : d->pack_events) cudaEventDestroy(e);
    d->pack_events.clear();
    d->ids_pinned = d->ids_device = nullptr;
    d->rows_device = nullptr;
    d->rows_host = nullptr;
    d->block_host = d->block_dev = d->all_dev = d->all_host = nullptr;
    d->staged = d->uploaded = d->queued = false;
}

// rank_of for all requests and every rank's run order: by length, then by request index.
int layout(const int* lengths, int n, int world, double a, double b, const double* speed, std::vector<int>& rank_of,
           std::vector<std::vector<int>>& members) {
    if (n < 0 || world <= 0 || (n > 0 && !lengths)) return S1_ERR_ARGUMENT;
    rank_of.assign(n, 0);
    D_TRY(s1_assign_requests_weighted(lengths, n, world, a, b, speed, rank_of.data()));
    members.assign(world, {});
    for (int i = 0; i < n; i++) members[rank_of[i]].push_back(i);
    for (auto& m : members)
        std::stable_sort(m.begin(), m.end(), [&](int x, int y) { return lengths[x] < lengths[y]; });
    return 0;
}

int read_id(const std::string& path, ncclUniqueId* id) {
    for (int tries = 0; tries < 2400; tries++) {  // two minutes
        FILE* f = fopen(path.c_str(), "rb");
        if (f) {
            const size_t got = fread(id, 1, sizeof(*id), f);
            fclose(f);
            if (got == sizeof(*id)) return 0;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    return S1_ERR_DISPATCH_RENDEZVOUS;
}

int write_id(const std::string& path, const ncclUniqueId& id) {
    const std::string tmp = path + ".part";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return S1_ERR_DISPATCH_RENDEZVOUS;
    const size_t put = fwrite(&id, 1, sizeof(id), f);
    if (fclose(f) != 0 || put != sizeof(id)) return S1_ERR_DISPATCH_RENDEZVOUS;
    return rename(tmp.c_str(), path.c_str()) == 0 ? 0 : S1_ERR_DISPATCH_RENDEZVOUS;  // appears whole or not at all
}

int side_room(Dispatch* d, size_t doubles) {
    if (d->side_cap >= doubles) return 0;
    if (d->side_dev) cudaFree(d->side_dev);
    d->side_dev = nullptr;
    d->side_cap = 0;
    D_TRY((int)cudaMalloc(reinterpret_cast<void**>(&d->side_dev), doubles * sizeof(double)));
    d->side_cap = doubles;
    return 0;
}

}  // namespace

extern "C" {

int s1_dispatch_layout(const int* lengths, int n, int world, double a, double b, int rank, int* rank_of,
                       int* local_index, int* n_local, int* pack_start) {
    return s1_dispatch_layout_weighted(lengths, n, world, a, b, nullptr, rank, rank_of, local_index, n_local, pack_start);
}

int s1_dispatch_layout_weighted(const int* lengths, int n, int world, double a, double b, const double* speed, int rank,
                                int* rank_of, int* local_index, int* n_local, int* pack_start) {
    if (rank < 0 || rank >= world) return -S1_ERR_ARGUMENT;
    std::vector<int> ranks;
    std::vector<std::vector<int>> members;
    const int rc = layout(lengths, n, world, a, b, speed, ranks, members);
    if (rc != 0) return -rc;
    if (rank_of) std::copy(ranks.begin(), ranks.end(), rank_of);
    const std::vector<int>& mine = members[rank];
    if (n_local) *n_local = (int)mine.size();
    if (local_index) std::copy(mine.begin(), mine.end(), local_index);
    std::vector<int> len(mine.size()), starts(mine.size() + 1);
    for (size_t i = 0; i < mine.size(); i++) len[i] = lengths[mine[i]];
    const int packs = s1_batch_ranges(len.data(), (int)len.size(), starts.data());
    if (pack_start) std::copy(starts.begin(), starts.begin() + packs, pack_start);
    return packs;
}

int s1_dispatch_create(int rank, int world, int device, const char* rendezvous, const char* nccl_library, void** out) {
    if (!out || world <= 0 || rank < 0 || rank >= world) return S1_ERR_ARGUMENT;
    D_TRY(cs1_set_device(device));
    Dispatch* d = new Dispatch();
    d->rank = rank;
    d->world = world;
    d->device = device;
    int rc = (int)cudaStreamCreateWithFlags(&d->side, cudaStreamNonBlocking);
    if (rc == 0 && world > 1) {
        rc = d->nccl.load(nccl_library);
        ncclUniqueId id;
        memset(&id, 0, sizeof(id));
        if (rc == 0 && (!rendezvous || !rendezvous[0])) rc = S1_ERR_ARGUMENT;
        if (rc == 0) {
            if (rank == 0) {
                rc = nccl_rc(d->nccl.GetUniqueId(&id));
                if (rc == 0) rc = write_id(rendezvous, id);
            } else {
                rc = read_id(rendezvous, &id);
            }
        }
        if (rc == 0) rc = nccl_rc(d->nccl.CommInitRank(&d->comm, world, id, rank));
        if (rank == 0 && rendezvous) unlink(rendezvous);  // every rank has joined, or the job has failed
    }
    if (rc != 0) {
        s1_dispatch_destroy(d);
        return rc;
    }
    *out = d;
    return 0;
}

void s1_dispatch_destroy(void* dispatch) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d) return;
    cs1_set_device(d->device);
    cudaDeviceSynchronize();
    release_plan(d);
    if (d->comm) d->nccl.CommDestroy(d->comm);
    if (d->side_dev) cudaFree(d->side_dev);
    if (d->side) cudaStreamDestroy(d->side);
    // libnccl stays loaded: unloading a library with live CUDA state is not safe
    delete d;
}

int s1_dispatch_set_cost(void* dispatch, double a, double b) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !(a >= 0.0) || !(b >= 0.0) || a + b <= 0.0) return S1_ERR_ARGUMENT;
    d->a = a;
    d->b = b;
    return 0;
}

int s1_dispatch_set_speed(void* dispatch, const double* speed, int world) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || (speed && world != d->world)) return S1_ERR_ARGUMENT;
    for (int r = 0; speed && r < world; r++)
        if (!(speed[r] > 0.0) || !std::isfinite(speed[r])) return S1_ERR_ARGUMENT;
    if (speed)
        d->speed.assign(speed, speed + world);
    else
        d->speed.clear();
    return 0;
}

int s1_dispatch_plan(void* dispatch, void* model, const int* lengths, int n, int n_classes) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !model || n <= 0 || !lengths || n_classes <= 0) return S1_ERR_ARGUMENT;
    S1Config cfg;
    D_TRY(s1_model_config(model, &cfg));
    D_TRY(cs1_set_device(d->device));
    D_TRY(s1_model_sync(model));
    release_plan(d);
    d->model = model;
    d->hidden = cfg.hidden;
    d->n_classes = n_classes;
    d->n = n;
    d->lengths.assign(lengths, lengths + n);
    D_TRY(layout(lengths, n, d->world, d->a, d->b, d->speed.empty() ? nullptr : d->speed.data(), d->rank_of, d->members));
    d->most = 0;
    for (const auto& m : d->members) d->most = std::max(d->most, (int)m.size());
    const std::vector<int>& mine = d->members[d->rank];
    d->local_len.resize(mine.size());
    d->token_at.resize(mine.size());
    d->local_tokens = 0;
    for (size_t i = 0; i < mine.size(); i++) {
        d->local_len[i] = lengths[mine[i]];
        d->token_at[i] = d->local_tokens;
        d->local_tokens += (size_t)lengths[mine[i]];
    }
    d->pack_start.assign(mine.size() + 1, 0);
    const int packs = s1_batch_ranges(d->local_len.data(), (int)mine.size(), d->pack_start.data());
    d->pack_start.resize(packs);
    long widest = 1;  // tokens of the largest pack: one scratch size for every pass
    for (int p = 0; p < packs; p++) {
        const int s0 = d->pack_start[p], s1 = p + 1 < packs ? d->pack_start[p + 1] : (int)mine.size();
        long t = 0;
        for (int i = s0; i < s1; i++) t += d->local_len[i];
        widest = std::max(widest, t);
    }
    D_TRY(s1_model_reserve(model, (int)widest));
    const size_t ids_bytes = std::max<size_t>(d->local_tokens, 1) * sizeof(int32_t);
    const size_t rows_bytes = std::max<size_t>(mine.size(), 1) * d->hidden * 2;
    const size_t block = (size_t)d->most * n_classes * sizeof(float);
    D_TRY((int)cudaHostAlloc(reinterpret_cast<void**>(&d->ids_pinned), ids_bytes, cudaHostAllocDefault));
    D_TRY((int)cudaMalloc(reinterpret_cast<void**>(&d->ids_device), ids_bytes));
    D_TRY((int)cudaMalloc(&d->rows_device, rows_bytes));
    D_TRY((int)cudaHostAlloc(reinterpret_cast<void**>(&d->rows_host), rows_bytes, cudaHostAllocDefault));
    D_TRY((int)cudaHostAlloc(reinterpret_cast<void**>(&d->block_host), block, cudaHostAllocDefault));
    D_TRY((int)cudaHostAlloc(reinterpret_cast<void**>(&d->all_host), block * d->world, cudaHostAllocDefault));
    D_TRY((int)cudaMalloc(reinterpret_cast<void**>(&d->block_dev), block));
    D_TRY((int)cudaMalloc(reinterpret_cast<void**>(&d->all_dev), block * d->world));
    d->pack_events.resize(2 * (size_t)packs);
    for (cudaEvent_t& e : d->pack_events) D_TRY((int)cudaEventCreate(&e));
    return 0;
}

int s1_dispatch_info(void* dispatch, int* n_local, long long* local_tokens, int* n_packs, int* rank_of) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !d->model) return S1_ERR_DISPATCH_STATE;
    if (n_local) *n_local = (int)d->local_len.size();
    if (local_tokens) *local_tokens = (long long)d->local_tokens;
    if (n_packs) *n_packs = (int)d->pack_start.size();
    if (rank_of) std::copy(d->rank_of.begin(), d->rank_of.end(), rank_of);
    return 0;
}

int s1_dispatch_local(void* dispatch, int* local_index, int* pack_start) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !d->model) return S1_ERR_DISPATCH_STATE;
    const std::vector<int>& mine = d->members[d->rank];
    if (local_index) std::copy(mine.begin(), mine.end(), local_index);
    if (pack_start) std::copy(d->pack_start.begin(), d->pack_start.end(), pack_start);
    return 0;
}

int s1_dispatch_stage(void* dispatch, const int32_t* ids_all) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !d->model) return S1_ERR_DISPATCH_STATE;
    if (!ids_all) return S1_ERR_ARGUMENT;
    D_TRY(cs1_set_device(d->device));
    D_TRY(s1_model_sync(d->model));  // no queued pass may still read the buffer
    std::vector<size_t> first(d->n + 1, 0);
    for (int i = 0; i < d->n; i++) first[i + 1] = first[i] + (size_t)d->lengths[i];
    const std::vector<int>& mine = d->members[d->rank];
    for (size_t i = 0; i < mine.size(); i++)
        memcpy(d->ids_pinned + d->token_at[i], ids_all + first[mine[i]], (size_t)d->local_len[i] * sizeof(int32_t));
    d->staged = true;
    d->uploaded = false;
    return 0;
}

int s1_dispatch_upload(void* dispatch) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !d->model || !d->staged) return S1_ERR_DISPATCH_STATE;
    D_TRY(cs1_set_device(d->device));
    if (d->local_tokens)
        D_TRY(cs1_upload(d->ids_device, d->ids_pinned, d->local_tokens * sizeof(int32_t), s1_model_stream(d->model)));
    d->uploaded = true;
    return 0;
}

int s1_dispatch_enqueue(void* dispatch, int resident) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !d->model || !d->staged || (resident && !d->uploaded)) return S1_ERR_DISPATCH_STATE;
    D_TRY(cs1_set_device(d->device));
    void* st = s1_model_stream(d->model);
    const int packs = (int)d->pack_start.size(), n_local = (int)d->local_len.size();
    for (int p = 0; p < packs; p++) {
        const int s0 = d->pack_start[p], s1 = p + 1 < packs ? d->pack_start[p + 1] : n_local;
        char* rows = static_cast<char*>(d->rows_device) + (size_t)s0 * d->hidden * 2;
        D_TRY(s1_event_record(d->pack_events[2 * p], st));
        if (resident) {
            void* last = nullptr;
            D_TRY(s1_model_forward_device(d->model, d->ids_device + d->token_at[s0], d->local_len.data() + s0, s1 - s0, &last));
            D_TRY(cs1_copy_dd(rows, last, (size_t)(s1 - s0) * d->hidden * 2, st));
        } else {
            D_TRY(s1_model_forward_queue(d->model, d->ids_pinned + d->token_at[s0], d->local_len.data() + s0, s1 - s0, rows));
        }
        D_TRY(s1_event_record(d->pack_events[2 * p + 1], st));
    }
    d->queued = true;
    return 0;
}

int s1_dispatch_pack_ms(void* dispatch, float* pack_ms) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !d->model || !d->queued) return S1_ERR_DISPATCH_STATE;
    if (!pack_ms) return S1_ERR_ARGUMENT;
    D_TRY(s1_model_sync(d->model));
    for (size_t p = 0; p < d->pack_start.size(); p++)
        D_TRY(s1_event_elapsed_ms(d->pack_events[2 * p], d->pack_events[2 * p + 1], &pack_ms[p]));
    return 0;
}

int s1_dispatch_collect(void* dispatch, const float* head_weights, const float* head_bias, float* logits,
                        double* gather_us) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !d->model || !d->queued) return S1_ERR_DISPATCH_STATE;
    if (!head_weights || (d->rank == 0 && !logits)) return S1_ERR_ARGUMENT;
    D_TRY(cs1_set_device(d->device));
    const int n_local = (int)d->local_len.size(), h = d->hidden, nc = d->n_classes;
    D_TRY(s1_model_read_rows(d->model, d->rows_host, d->rows_device, (size_t)n_local * h * 2));
    d->queued = false;
    std::vector<float> last(h);
    const size_t block = (size_t)d->most * nc;
    std::fill(d->block_host, d->block_host + block, 0.f);
    for (int i = 0; i < n_local; i++) {
        const uint16_t* row = d->rows_host + (size_t)i * h;
        for (int j = 0; j < h; j++) {
            const uint32_t u = (uint32_t)row[j] << 16;
            memcpy(&last[j], &u, 4);
        }
        D_TRY(s1_head_logits(head_weights, head_bias, last.data(), h, nc, d->block_host + (size_t)i * nc));
    }
    const float* all = d->block_host;
    const auto t0 = std::chrono::steady_clock::now();
    if (d->world > 1) {
        cudaStream_t st = static_cast<cudaStream_t>(s1_model_stream(d->model));
        D_TRY((int)cudaMemcpyAsync(d->block_dev, d->block_host, block * sizeof(float), cudaMemcpyHostToDevice, st));
        D_TRY(nccl_rc(d->nccl.AllGather(d->block_dev, d->all_dev, block, ncclFloat32, d->comm, st)));
        if (d->rank == 0)
            D_TRY((int)cudaMemcpyAsync(d->all_host, d->all_dev, block * d->world * sizeof(float), cudaMemcpyDeviceToHost, st));
        D_TRY((int)cudaStreamSynchronize(st));
        all = d->all_host;
    }
    if (gather_us)
        *gather_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    if (d->rank == 0) {
        for (int r = 0; r < d->world; r++) {
            const std::vector<int>& theirs = d->members[r];
            for (size_t i = 0; i < theirs.size(); i++)
                memcpy(logits + (size_t)theirs[i] * nc, all + ((size_t)r * d->most + i) * nc, (size_t)nc * sizeof(float));
        }
    }
    return 0;
}

int s1_dispatch_candidates(void* dispatch, void* model, const void* prefix, const int32_t* ids, const int* lengths, int n,
                           const float* head_weights, const float* head_bias, int n_classes, float* logits,
                           int* rank_of_out) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || !model || !prefix || !ids || !lengths || n <= 0 || n_classes <= 0 || !head_weights ||
        (d->rank == 0 && !logits))
        return S1_ERR_ARGUMENT;
    S1Config cfg;
    D_TRY(s1_model_config(model, &cfg));
    D_TRY(cs1_set_device(d->device));
    // every candidate costs its own tokens (the prefix is there already on every rank)
    std::vector<int> rank_of;
    std::vector<std::vector<int>> members;
    D_TRY(layout(lengths, n, d->world, 1.0, 0.0, d->speed.empty() ? nullptr : d->speed.data(), rank_of, members));
    if (rank_of_out) std::copy(rank_of.begin(), rank_of.end(), rank_of_out);
    std::vector<size_t> first(n + 1, 0);
    for (int i = 0; i < n; i++) {
        if (lengths[i] <= 0) return S1_ERR_ARGUMENT;
        first[i + 1] = first[i] + (size_t)lengths[i];
    }
    int most = 0;
    for (const auto& m : members) most = std::max(most, (int)m.size());
    const std::vector<int>& mine = members[d->rank];
    // this rank's candidates, packed like requests (at most 16 prompts / 4096 tokens a pass)
    std::vector<int> len(mine.size()), starts(mine.size() + 1);
    for (size_t i = 0; i < mine.size(); i++) len[i] = lengths[mine[i]];
    const int packs = s1_batch_ranges(len.data(), (int)len.size(), starts.data());
    std::vector<double> block((size_t)most * n_classes, 0.0);
    std::vector<float> hidden, row(n_classes);
    std::vector<int32_t> pack_ids;
    for (int p = 0; p < packs; p++) {
        const int s0 = starts[p], s1 = p + 1 < packs ? starts[p + 1] : (int)mine.size();
        pack_ids.clear();
        for (int i = s0; i < s1; i++) pack_ids.insert(pack_ids.end(), ids + first[mine[i]], ids + first[mine[i] + 1]);
        hidden.resize((size_t)(s1 - s0) * cfg.hidden);
        D_TRY(s1_model_forward_continue(model, prefix, pack_ids.data(), len.data() + s0, s1 - s0, hidden.data()));
        for (int i = s0; i < s1; i++) {
            D_TRY(s1_head_logits(head_weights, head_bias, hidden.data() + (size_t)(i - s0) * cfg.hidden, cfg.hidden, n_classes,
                                 row.data()));
            for (int c = 0; c < n_classes; c++) block[(size_t)i * n_classes + c] = row[c];
        }
    }
    // float32 logits travel as float64 (exact) through the harness all-gather
    std::vector<double> all(block.size() * d->world);
    if (block.empty()) return 0;
    D_TRY(s1_dispatch_allgather(d, block.data(), (int)block.size(), all.data()));
    if (d->rank == 0)
        for (int r = 0; r < d->world; r++)
            for (size_t i = 0; i < members[r].size(); i++)
                for (int c = 0; c < n_classes; c++)
                    logits[(size_t)members[r][i] * n_classes + c] = (float)all[((size_t)r * most + i) * n_classes + c];
    return 0;
}

int s1_dispatch_barrier(void* dispatch) {
    double x = 0.0;
    return s1_dispatch_allreduce_max(dispatch, &x, 1);
}

int s1_dispatch_allreduce_max(void* dispatch, double* values, int n) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || n <= 0 || !values) return S1_ERR_ARGUMENT;
    D_TRY(cs1_set_device(d->device));
    D_TRY((int)cudaDeviceSynchronize());
    if (d->world == 1) return 0;
    D_TRY(side_room(d, (size_t)n));
    D_TRY((int)cudaMemcpyAsync(d->side_dev, values, n * sizeof(double), cudaMemcpyHostToDevice, d->side));
    D_TRY(nccl_rc(d->nccl.AllReduce(d->side_dev, d->side_dev, (size_t)n, ncclFloat64, ncclMax, d->comm, d->side)));
    D_TRY((int)cudaMemcpyAsync(values, d->side_dev, n * sizeof(double), cudaMemcpyDeviceToHost, d->side));
    return (int)cudaStreamSynchronize(d->side);
}

int s1_dispatch_allgather(void* dispatch, const double* values, int n, double* all) {
    Dispatch* d = static_cast<Dispatch*>(dispatch);
    if (!d || n <= 0 || !values || !all) return S1_ERR_ARGUMENT;
    D_TRY(cs1_set_device(d->device));
    if (d->world == 1) {
        memcpy(all, values, n * sizeof(double));
        return 0;
    }
    D_TRY(side_room(d, (size_t)n * (d->world + 1)));
    double* in = d->side_dev + (size_t)n * d->world;
    D_TRY((int)cudaMemcpyAsync(in, values, n * sizeof(double), cudaMemcpyHostToDevice, d->side));
    D_TRY(nccl_rc(d->nccl.AllGather(in, d->side_dev, (size_t)n, ncclFloat64, d->comm, d->side)));
    D_TRY((int)cudaMemcpyAsync(all, d->side_dev, (size_t)n * d->world * sizeof(double), cudaMemcpyDeviceToHost, d->side));
    return (int)cudaStreamSynchronize(d->side);
}

}  // extern "C"
