// Expert residency runtime: the LRU bookkeeping of the reference's ExpertCache
// (expert_cache.py:12-52, :93-201) plus a copy engine built for a machine where
// host memory is plentiful and the copy engines run beside the SMs:
//
//   * every expert keeps a pinned host copy for its whole life, so evicting one
//     is bookkeeping only (the reference copies the evicted slab back to the host,
//     expert_cache.py:189, although weights never change);
//   * host->device copies go to a side stream; an event per device slab orders
//     "copy finished" before the compute stream reads it and "last compute
//     enqueued" before the copy stream overwrites it (the reference issues both
//     copies on the compute stream, expert_cache.py:188-189);
//   * a slab whose expert was evicted while still waiting to be yielded in the
//     running request is never chosen as a copy target (the reference can hand
//     out such a slab after overwriting it when few buffers are configured).
//
// Which expert is resident, the yield order, hits and misses follow the
// reference step for step; the CPU tests replay its recorded traces.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include <algorithm>
#include <deque>
#include <list>
#include <map>
#include <new>
#include <unordered_map>
#include <vector>

#include "../../include/hqq_moe.h"

namespace hqm {
void set_error(const char* fmt, ...);
}

namespace {

struct Expert {
    int64_t uid;
    int32_t group;
    bool offloaded;
    int32_t index;          // logical main / offload slot, as ExpertInfo.index
    int32_t slab;           // physical device slab holding its bytes, -1 if none
    const void* host;       // pinned host copy
    bool prefetched = false;   // brought in by hqm_cache_prefetch and not requested since
};

struct Group {
    std::list<int64_t> main_lru;   // least recently used first (EvictionGroupInfo.main_infos)
    std::list<int64_t> off_lru;    // EvictionGroupInfo.offloaded_infos
    int64_t hits = 0, misses = 0;
};

struct Slab {
    void* ptr = nullptr;
    int64_t holder = -1;           // uid whose bytes are (being) stored here
    bool pending = false;          // holder was requested in the running call and not yielded yet
    bool copy_in_flight = false;   // compute stream has not yet waited for `ready`
    bool used = false;             // `last_use` has been recorded at least once
    cudaEvent_t ready = nullptr, last_use = nullptr;
};

}  // namespace

struct hqm_cache {
    int32_t main_size, offload_size, buffer_size, device_id;
    size_t slab_bytes;
    bool with_cuda;
    cudaStream_t copy_stream = nullptr;
    std::vector<Slab> slabs;                 // main_size + buffer_size physical device slabs
    std::deque<int32_t> free_slabs;          // spare slabs, next copy target first
    std::vector<int64_t> main_slots, off_slots;   // logical slots -> uid or -1
    std::unordered_map<int64_t, Expert> experts;
    std::map<int32_t, Group> groups;
    int64_t h2d_bytes = 0, swaps = 0;
    int64_t prefetch_issued = 0, prefetch_used = 0, prefetch_wasted = 0;
    // state of the running request
    bool active = false;
    int32_t cur_group = 0;
    std::vector<int64_t> order;
    std::deque<int64_t> pre_loaded, to_load, in_loading;
    size_t pos = 0;
    int32_t current_slab = -1;               // slab of the expert handed out last
    bool swap_on_resume = false;             // the expert handed out last came from a copy of this request
};

namespace {

#define CACHE_CUDA(c, call)                                                                      \
    do {                                                                                         \
        cudaError_t e_ = (call);                                                                 \
        if (e_ != cudaSuccess) {                                                                 \
            hqm::set_error("%s failed: %s", #call, cudaGetErrorString(e_));                      \
            return HQM_ERR_CUDA;                                                                 \
        }                                                                                        \
    } while (0)

int state_error(const char* fmt, ...) {
    char buf[400];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    hqm::set_error("%s", buf);
    return HQM_ERR_STATE;
}

// Queue the host->device copy of `e` into slab `s` on the copy stream.
int issue_copy(hqm_cache* c, Expert& e, int32_t s, bool count_as_swap) {
    Slab& sl = c->slabs[s];
    sl.holder = e.uid;
    e.slab = s;
    if (count_as_swap) c->h2d_bytes += (int64_t)c->slab_bytes;
    if (!c->with_cuda) return HQM_OK;
    if (sl.used) CACHE_CUDA(c, cudaStreamWaitEvent(c->copy_stream, sl.last_use, 0));
    CACHE_CUDA(c, cudaMemcpyAsync(sl.ptr, e.host, c->slab_bytes, cudaMemcpyHostToDevice, c->copy_stream));
    CACHE_CUDA(c, cudaEventRecord(sl.ready, c->copy_stream));
    sl.copy_in_flight = true;
    return HQM_OK;
}

// _swap, expert_cache.py:181-201: `uid_in` becomes resident, the group's least
// recently used resident expert leaves.
int swap_in(hqm_cache* c, Group& g, int64_t uid_in) {
    if (g.main_lru.empty()) return state_error("No evictable experts");
    // a spare slab that is safe to overwrite (position in the spare queue)
    int target = -1;
    for (size_t i = 0; i < c->free_slabs.size() && target < 0; ++i)
        if (!c->slabs[c->free_slabs[i]].pending) target = (int)i;
    // victim: the least recently used; if no spare slab is safe, the least recently
    // used expert that is not itself waiting to be yielded (its slab becomes the target)
    auto victim_it = g.main_lru.begin();
    if (target < 0) {
        for (; victim_it != g.main_lru.end(); ++victim_it) {
            const Expert& v = c->experts.at(*victim_it);
            if (!c->slabs[v.slab].pending) break;
        }
        if (victim_it == g.main_lru.end())
            return state_error("no device buffer can be overwritten: every spare slab holds an expert that is still "
                               "waiting to be yielded");
    }
    Expert& in = c->experts.at(uid_in);
    Expert& out = c->experts.at(*victim_it);
    if (!in.offloaded || out.offloaded || in.group != out.group) return state_error("internal error: bad swap");

    c->free_slabs.push_back(out.slab);          // its bytes stay valid until the slab is reused
    if (target < 0) target = (int)c->free_slabs.size() - 1;
    const int32_t s = c->free_slabs[target];
    c->free_slabs.erase(c->free_slabs.begin() + target);

    // bookkeeping exactly as the reference: exchange logical slots and flags
    c->main_slots[out.index] = in.uid;
    c->off_slots[in.index] = out.uid;
    std::swap(in.index, out.index);
    in.offloaded = false;
    out.offloaded = true;
    out.slab = -1;
    if (out.prefetched) {                       // a guess that was never asked for leaves again
        out.prefetched = false;
        c->prefetch_wasted += 1;
    }
    g.off_lru.remove(in.uid);
    g.main_lru.push_back(in.uid);               // most recently used
    g.main_lru.erase(victim_it);
    g.off_lru.push_back(out.uid);
    c->swaps += 1;
    return issue_copy(c, in, s, /*count_as_swap=*/true);
}

int finish_current(hqm_cache* c, void* compute_stream) {
    if (c->current_slab >= 0 && c->with_cuda) {
        Slab& sl = c->slabs[c->current_slab];
        CACHE_CUDA(c, cudaEventRecord(sl.last_use, (cudaStream_t)compute_stream));
        sl.used = true;
    }
    c->current_slab = -1;
    return HQM_OK;
}

}  // namespace

extern "C" {

int hqm_cache_create(hqm_cache** out, int32_t main_size, int32_t offload_size, int32_t buffer_size, size_t slab_bytes,
                     void* const* device_slabs, int32_t device_id) {
    if (!out || main_size < 0 || offload_size < 0 || buffer_size < 0) {
        hqm::set_error("cache_create: bad sizes (%d, %d, %d)", main_size, offload_size, buffer_size);
        return HQM_ERR_ARG;
    }
    hqm_cache* c = new (std::nothrow) hqm_cache();
    if (!c) {
        hqm::set_error("cache_create: out of host memory");
        return HQM_ERR_ARG;
    }
    c->main_size = main_size;
    c->offload_size = offload_size;
    c->buffer_size = buffer_size;
    c->device_id = device_id;
    c->slab_bytes = slab_bytes;
    c->with_cuda = device_slabs != nullptr;
    c->slabs.resize((size_t)main_size + buffer_size);
    c->main_slots.assign(main_size, -1);
    c->off_slots.assign(offload_size, -1);
    for (int32_t i = 0; i < main_size + buffer_size; ++i) c->free_slabs.push_back(i);
    if (c->with_cuda) {
        cudaError_t e = cudaSetDevice(device_id);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking);
        for (size_t i = 0; e == cudaSuccess && i < c->slabs.size(); ++i) {
            c->slabs[i].ptr = device_slabs[i];
            e = cudaEventCreateWithFlags(&c->slabs[i].ready, cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->slabs[i].last_use, cudaEventDisableTiming);
        }
        if (e != cudaSuccess) {
            hqm::set_error("cache_create: %s", cudaGetErrorString(e));
            hqm_cache_destroy(c);
            return HQM_ERR_CUDA;
        }
    }
    *out = c;
    return HQM_OK;
}

void hqm_cache_destroy(hqm_cache* c) {
    if (!c) return;
    if (c->with_cuda) {
        if (c->copy_stream) cudaStreamSynchronize(c->copy_stream);
        for (auto& s : c->slabs) {
            if (s.ready) cudaEventDestroy(s.ready);
            if (s.last_use) cudaEventDestroy(s.last_use);
        }
        if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    }
    delete c;
}

int hqm_cache_add(hqm_cache* c, int64_t uid, int32_t eviction_group, int32_t offload, const void* host_slab,
                  int32_t* placed_offloaded, void* stream) {
    (void)stream;
    if (!c) return state_error("cache_add: null handle");
    if (c->active) return state_error("already loading experts; buffers are busy");
    if (c->experts.count(uid)) return state_error("expert %lld already registered", (long long)uid);
    if (c->with_cuda && !host_slab) return state_error("cache_add: the pinned host copy is required");
    Expert e{uid, eviction_group, false, -1, -1, host_slab};
    bool placed = false;
    if (offload != 1) {   // False or None: first free device slot
        for (int32_t i = 0; i < c->main_size && !placed; ++i)
            if (c->main_slots[i] < 0) {
                c->main_slots[i] = uid;
                e.index = i;
                e.offloaded = false;
                placed = true;
            }
    }
    if (!placed && offload != 0) {   // True or None: first free host slot
        for (int32_t i = 0; i < c->offload_size && !placed; ++i)
            if (c->off_slots[i] < 0) {
                c->off_slots[i] = uid;
                e.index = i;
                e.offloaded = true;
                placed = true;
            }
    }
    if (!placed) return state_error("Cache is full");
    Group& g = c->groups[eviction_group];
    auto ins = c->experts.emplace(uid, e);
    if (e.offloaded) {
        g.off_lru.push_back(uid);
    } else {
        g.main_lru.push_back(uid);
        const int32_t s = c->free_slabs.front();
        c->free_slabs.pop_front();
        int rc = issue_copy(c, ins.first->second, s, /*count_as_swap=*/false);
        if (rc != HQM_OK) return rc;
    }
    if (placed_offloaded) *placed_offloaded = e.offloaded ? 1 : 0;
    return HQM_OK;
}

int hqm_cache_begin(hqm_cache* c, const int64_t* uids, int32_t n, int32_t unordered, int64_t* order_out,
                    void* compute_stream) {
    (void)compute_stream;
    if (!c || (n > 0 && !uids)) return state_error("cache_begin: null argument");
    if (c->active) return state_error("already loading experts; buffers are busy");
    std::vector<int64_t> req(uids, uids + n);
    {
        std::vector<int64_t> sorted = req;
        std::sort(sorted.begin(), sorted.end());
        if (std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end())
            return state_error("load_experts: duplicate uids");
    }
    for (int64_t u : req)
        if (!c->experts.count(u)) return state_error("load_experts: expert %lld is not registered", (long long)u);
    c->order.clear();
    c->pre_loaded.clear();
    c->to_load.clear();
    c->in_loading.clear();
    c->pos = 0;
    c->current_slab = -1;
    c->swap_on_resume = false;
    if (n == 0) {
        c->active = true;
        return HQM_OK;
    }
    if (unordered)   // resident experts first, otherwise in the order given
        std::stable_sort(req.begin(), req.end(), [&](int64_t a, int64_t b) {
            return (int)c->experts.at(a).offloaded < (int)c->experts.at(b).offloaded;
        });
    const int32_t group = c->experts.at(req[0]).group;
    for (int64_t u : req)
        if (c->experts.at(u).group != group) return state_error("experts must be in the same evicton group");
    Group& g = c->groups[group];
    for (int64_t u : req) {   // mark_used, expert_cache.py:44-52
        Expert& e = c->experts.at(u);
        if (e.prefetched) {   // the guess was right: what would have been a miss is a hit
            e.prefetched = false;
            c->prefetch_used += 1;
        }
        std::list<int64_t>& l = e.offloaded ? g.off_lru : g.main_lru;
        l.remove(u);
        l.push_back(u);
        if (e.offloaded) g.misses += 1; else g.hits += 1;
    }
    c->active = true;
    c->cur_group = group;
    c->order = req;
    for (int64_t u : req) {
        Expert& e = c->experts.at(u);
        if (e.offloaded) {
            c->to_load.push_back(u);
        } else {
            c->pre_loaded.push_back(u);
            c->slabs[e.slab].pending = true;
        }
    }
    if (order_out) std::copy(req.begin(), req.end(), order_out);
    const int32_t window = std::min<int32_t>(
        std::min<int32_t>(c->buffer_size - 1, (int32_t)g.main_lru.size()), (int32_t)c->to_load.size());
    for (int32_t i = 0; i < window; ++i) {
        const int64_t u = c->to_load.front();
        c->to_load.pop_front();
        c->in_loading.push_back(u);
        int rc = swap_in(c, g, u);
        if (rc != HQM_OK) {
            hqm_cache_end(c, compute_stream);
            return rc;
        }
        c->slabs[c->experts.at(u).slab].pending = true;
    }
    return HQM_OK;
}

int hqm_cache_next(hqm_cache* c, int64_t* uid_out, void** slab_out, int32_t* slot_out, void* compute_stream) {
    if (!c) return state_error("cache_next: null handle");
    if (!c->active) return state_error("cache_next: no request is running");
    Group& g = c->groups[c->cur_group];
    // the consumer is back: the expert handed out last has had its compute enqueued
    int rc = finish_current(c, compute_stream);
    if (rc != HQM_OK) return rc;
    if (c->swap_on_resume) {   // expert_cache.py:171-175: a loaded expert was consumed, start the next copy
        c->swap_on_resume = false;
        if (!c->to_load.empty()) {
            const int64_t nxt = c->to_load.front();
            c->to_load.pop_front();
            c->in_loading.push_back(nxt);
            rc = swap_in(c, g, nxt);
            if (rc != HQM_OK) {
                hqm_cache_end(c, compute_stream);
                return rc;
            }
            c->slabs[c->experts.at(nxt).slab].pending = true;
        }
    }
    if (c->pos >= c->order.size()) {
        hqm_cache_end(c, compute_stream);
        return 1;
    }
    const int64_t u = c->order[c->pos];
    int32_t s = -1;
    bool was_loading = false;
    if (!c->pre_loaded.empty() && c->pre_loaded.front() == u) {
        c->pre_loaded.pop_front();
    } else if (!c->in_loading.empty() && c->in_loading.front() == u) {
        c->in_loading.pop_front();
        was_loading = true;
    } else {
        hqm_cache_end(c, compute_stream);
        return state_error("internal error: caching algorithm failed");
    }
    // A pre-loaded expert may have been evicted by a swap of this very request; its
    // bytes are still in the slab it occupied when the request began.
    for (size_t i = 0; i < c->slabs.size() && s < 0; ++i)
        if (c->slabs[i].holder == u && c->slabs[i].pending) s = (int32_t)i;
    if (s < 0) {
        hqm_cache_end(c, compute_stream);
        return state_error("internal error: expert %lld has no device slab", (long long)u);
    }
    Slab& sl = c->slabs[s];
    sl.pending = false;
    if (c->with_cuda && sl.copy_in_flight) {
        CACHE_CUDA(c, cudaStreamWaitEvent((cudaStream_t)compute_stream, sl.ready, 0));
        sl.copy_in_flight = false;
    }
    c->current_slab = s;
    c->pos += 1;
    if (uid_out) *uid_out = u;
    if (slab_out) *slab_out = sl.ptr;
    if (slot_out) *slot_out = s;
    c->swap_on_resume = was_loading;
    return HQM_OK;
}

int hqm_cache_end(hqm_cache* c, void* compute_stream) {
    if (!c) return state_error("cache_end: null handle");
    int rc = finish_current(c, compute_stream);
    for (auto& s : c->slabs) s.pending = false;
    c->active = false;
    c->swap_on_resume = false;
    c->order.clear();
    c->pre_loaded.clear();
    c->to_load.clear();
    c->in_loading.clear();
    c->pos = 0;
    return rc;
}

// Speculative loading, which the reference lists as not yet implemented (README.md:24-27): outside a request,
// bring experts that are expected to be asked for soon onto the device, exactly as a miss would (the group's least
// recently used resident expert leaves, the copy runs on the side stream), but without counting a hit or a miss
// and without touching the order of experts that are already resident.
int hqm_cache_prefetch(hqm_cache* c, const int64_t* uids, int32_t n, int32_t* issued_out) {
    if (!c || (n > 0 && !uids)) return state_error("cache_prefetch: null argument");
    if (c->active) return state_error("already loading experts; buffers are busy");
    int32_t issued = 0;
    for (int32_t i = 0; i < n; ++i) {
        auto it = c->experts.find(uids[i]);
        if (it == c->experts.end()) return state_error("cache_prefetch: expert %lld is not registered", (long long)uids[i]);
        Expert& e = it->second;
        if (!e.offloaded) continue;
        Group& g = c->groups[e.group];
        if (g.main_lru.empty()) continue;
        const int rc = swap_in(c, g, e.uid);
        if (rc != HQM_OK) return rc;
        e.prefetched = true;
        c->prefetch_issued += 1;
        ++issued;
    }
    if (issued_out) *issued_out = issued;
    return HQM_OK;
}

int hqm_cache_prefetch_stats(hqm_cache* c, int64_t* issued, int64_t* used, int64_t* wasted) {
    if (!c) return state_error("cache_prefetch_stats: null handle");
    if (issued) *issued = c->prefetch_issued;
    if (used) *used = c->prefetch_used;
    if (wasted) *wasted = c->prefetch_wasted;
    return HQM_OK;
}

int hqm_cache_stats(hqm_cache* c, int32_t eviction_group, int64_t* hits, int64_t* misses, int64_t* h2d_bytes,
                    int64_t* swaps) {
    if (!c) return state_error("cache_stats: null handle");
    auto it = c->groups.find(eviction_group);
    if (hits) *hits = it == c->groups.end() ? 0 : it->second.hits;
    if (misses) *misses = it == c->groups.end() ? 0 : it->second.misses;
    if (h2d_bytes) *h2d_bytes = c->h2d_bytes;
    if (swaps) *swaps = c->swaps;
    return HQM_OK;
}

int hqm_cache_resident(hqm_cache* c, int32_t eviction_group, int64_t* uids_out, int32_t cap) {
    if (!c) return 0;
    auto it = c->groups.find(eviction_group);
    if (it == c->groups.end()) return 0;
    int32_t n = 0;
    for (int64_t u : it->second.main_lru) {
        if (uids_out && n < cap) uids_out[n] = u;
        ++n;
    }
    return n;
}

}  // extern "C"
