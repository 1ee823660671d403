// Host storage for evicted tensors: gpu_storage_t (src/engine/gpu/storage.{h,cc}) and the
// evict / load exec nodes (src/engine/gpu/exec_graph.cc:469-577) behind the C ABI.
//
// One pinned, portable host arena per storage (the reference's cudaHostAlloc of the whole
// storage_size, storage.cc:4-29); every storage id owns one block of it, found first-fit.
// es_b200_evict reserves the id's block and issues one cudaMemcpyAsync device -> host;
// es_b200_load issues the copy back and -- where the reference removes the id from a stream
// callback once the copy has finished -- records an event: the block returns to the free list
// when that event has completed, checked whenever a later call needs space.
#include <cuda_runtime.h>

#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "common.h"
#include "handle.h"

struct es_b200_storage {
    char*      base = nullptr;
    uint64_t   bytes = 0;
    std::mutex m;
    struct block_t {
        uint64_t offset, size;
    };
    std::map<int, block_t>       info;      // id -> block
    std::map<uint64_t, uint64_t> free_list; // offset -> size, coalesced
    struct pending_t {
        cudaEvent_t event;
        block_t     block;
    };
    std::vector<pending_t> pending; // loads in flight whose blocks are not free yet
};

namespace {

using namespace es;

template <typename F> int guarded(F&& f)
{
    try {
        f();
        return ES_OK;
    } catch (es_error const& e) {
        set_last_error(e.what());
        return e.status;
    } catch (std::exception const& e) {
        set_last_error(e.what());
        return ES_BAD_ARGUMENT;
    }
}

void give_back(es_b200_storage* s, es_b200_storage::block_t b)
{
    auto it = s->free_list.emplace(b.offset, b.size).first;
    auto next = std::next(it);
    if (next != s->free_list.end() && it->first + it->second == next->first) {
        it->second += next->second;
        s->free_list.erase(next);
    }
    if (it != s->free_list.begin()) {
        auto prev = std::prev(it);
        if (prev->first + prev->second == it->first) {
            prev->second += it->second;
            s->free_list.erase(it);
        }
    }
}

void reap(es_b200_storage* s, bool wait)
{
    for (size_t i = 0; i != s->pending.size();) {
        cudaError_t e = wait ? cudaEventSynchronize(s->pending[i].event) : cudaEventQuery(s->pending[i].event);
        if (e == cudaSuccess) {
            cudaEventDestroy(s->pending[i].event);
            give_back(s, s->pending[i].block);
            s->pending[i] = s->pending.back();
            s->pending.pop_back();
        } else {
            if (e != cudaErrorNotReady) cudaGetLastError();
            ++i;
        }
    }
}

es_b200_storage::block_t take(es_b200_storage* s, uint64_t size, int id)
{
    if (s->info.count(id)) fail(ES_BAD_ARGUMENT, "storage: id " + std::to_string(id) + " already in storage");
    uint64_t need = (size + 255) / 256 * 256;
    // first fit; when nothing fits, first collect the blocks of loads that have finished, then wait
    // for those still in flight
    for (int attempt = 0; attempt != 3; ++attempt) {
        if (attempt == 1) reap(s, false);
        if (attempt == 2) reap(s, true);
        for (auto it = s->free_list.begin(); it != s->free_list.end(); ++it) {
            if (it->second >= need) {
                uint64_t off = it->first, rest = it->second - need;
                s->free_list.erase(it);
                if (rest) s->free_list.emplace(off + need, rest);
                s->info[id] = es_b200_storage::block_t{off, size};
                return es_b200_storage::block_t{off, need};
            }
        }
    }
    fail(ES_WORKSPACE_TOO_SMALL, "storage: ran out of space for " + std::to_string(size) + " bytes");
}

es_b200_storage::block_t find(es_b200_storage* s, int id)
{
    auto it = s->info.find(id);
    if (it == s->info.end()) fail(ES_BAD_ARGUMENT, "storage: id " + std::to_string(id) + " not in storage");
    return it->second;
}

} // namespace

extern "C" {

int es_b200_storage_create(uint64_t bytes, int write_combined, es_b200_storage_t** out)
{
    return guarded([&] {
        if (!out || bytes == 0) fail(ES_BAD_ARGUMENT, "storage: null pointer or zero size");
        auto* s = new es_b200_storage;
        s->bytes = (bytes + 255) / 256 * 256;
        unsigned flags = cudaHostAllocPortable | (write_combined ? cudaHostAllocWriteCombined : 0);
        cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&s->base), s->bytes, flags);
        if (e != cudaSuccess) {
            delete s;
            fail(ES_CUDA_ERROR, std::string("cudaHostAlloc: ") + cudaGetErrorString(e));
        }
        s->free_list.emplace(0, s->bytes);
        *out = s;
    });
}

int es_b200_storage_destroy(es_b200_storage_t* s)
{
    return guarded([&] {
        if (!s) return;
        reap(s, true);
        cudaFreeHost(s->base);
        delete s;
    });
}

int es_b200_storage_write(es_b200_storage_t* s, int id, const void* host_src, uint64_t bytes)
{
    return guarded([&] {
        if (!s || !host_src) fail(ES_BAD_ARGUMENT, "storage: null pointer");
        std::lock_guard<std::mutex> lock(s->m);
        auto                        b = take(s, bytes, id);
        std::memcpy(s->base + b.offset, host_src, bytes);
    });
}

int es_b200_storage_read(es_b200_storage_t* s, int id, void* host_dst, uint64_t bytes)
{
    return guarded([&] {
        if (!s || !host_dst) fail(ES_BAD_ARGUMENT, "storage: null pointer");
        std::lock_guard<std::mutex> lock(s->m);
        auto                        b = find(s, id);
        if (b.size != bytes) fail(ES_BAD_ARGUMENT, "storage: id holds " + std::to_string(b.size) + " bytes");
        std::memcpy(host_dst, s->base + b.offset, bytes);
    });
}

int es_b200_storage_remove(es_b200_storage_t* s, int id)
{
    return guarded([&] {
        if (!s) fail(ES_BAD_ARGUMENT, "storage: null pointer");
        std::lock_guard<std::mutex> lock(s->m);
        auto                        b = find(s, id);
        s->info.erase(id);
        give_back(s, {b.offset, (b.size + 255) / 256 * 256});
    });
}

int es_b200_storage_reference(es_b200_storage_t* s, int id, void** host_ptr, uint64_t* bytes)
{
    return guarded([&] {
        if (!s || !host_ptr) fail(ES_BAD_ARGUMENT, "storage: null pointer");
        std::lock_guard<std::mutex> lock(s->m);
        auto                        b = find(s, id);
        *host_ptr = s->base + b.offset;
        if (bytes) *bytes = b.size;
    });
}

int es_b200_evict(es_b200_t* h, es_b200_storage_t* s, int id, const void* dev_src, uint64_t bytes, void* stream)
{
    return guarded([&] {
        if (!h || !s || !dev_src) fail(ES_BAD_ARGUMENT, "evict: null pointer");
        ES_CUDA_CHECK(cudaSetDevice(h->device));
        std::lock_guard<std::mutex> lock(s->m);
        auto                        b = take(s, bytes, id);
        ES_CUDA_CHECK(cudaMemcpyAsync(s->base + b.offset, dev_src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
        h->counters[3] += 1;
        h->work_bytes[3] += bytes;
    });
}

int es_b200_load(es_b200_t* h, es_b200_storage_t* s, int id, void* dev_dst, uint64_t bytes, void* stream)
{
    return guarded([&] {
        if (!h || !s || !dev_dst) fail(ES_BAD_ARGUMENT, "load: null pointer");
        ES_CUDA_CHECK(cudaSetDevice(h->device));
        std::lock_guard<std::mutex> lock(s->m);
        auto                        b = find(s, id);
        if (b.size != bytes) fail(ES_BAD_ARGUMENT, "load: id holds " + std::to_string(b.size) + " bytes");
        ES_CUDA_CHECK(cudaMemcpyAsync(dev_dst, s->base + b.offset, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
        // the id leaves the storage now; its bytes stay until the copy has finished
        es_b200_storage::pending_t p;
        ES_CUDA_CHECK(cudaEventCreateWithFlags(&p.event, cudaEventDisableTiming));
        ES_CUDA_CHECK(cudaEventRecord(p.event, (cudaStream_t)stream));
        p.block = {b.offset, (b.size + 255) / 256 * 256};
        s->pending.push_back(p);
        s->info.erase(id);
        h->counters[3] += 1;
        h->work_bytes[3] += bytes;
    });
}

} // extern "C"
