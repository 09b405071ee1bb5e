// C wrapper around the reference's own integer-side objects — TEST INFRASTRUCTURE ONLY.
//
// build_ref.py compiles this file together with the reference's own src/core/{req,batch,
// sampling_params}.cc, src/kernels/radix.cc, src/kvcache/{radix_tree,cache_manager}.cc and
// src/scheduler/{decode,prefill}.cc (taken from the reference tree where they lie, never copied)
// against the LibTorch inside the torch wheel.  What the wrapper adds:
//
//  * host definitions of write_token_pool / gather_int32_2d with the semantics of the reference's
//    CUDA kernels (src/kernels/token_pool.cu:10-49: out-of-range rows or positions are skipped on
//    write and read as 0), because CacheManager::write_page_table calls the former
//    (src/scheduler/prefill.cc:186) and the page table lives in host memory here;
//  * `HostScheduler`: the reference's TableManager, CacheManager, DecodeManager and PrefillManager
//    driven in the order of Scheduler::step_no_overlap (src/scheduler/scheduler.cc:275-358,365-389,
//    424-470,574-580) with the forward pass replaced by tokens the caller supplies;
//  * entry points on RadixPrefixCache, RadixTreeNode, Req and fast_compare_key so that the known
//    answers of the reference's own unit tests can be replayed from Python.
//
// CacheManager::ensure_page_write_workspace allocates PINNED host tensors, which needs a CUDA
// driver.  Its early return (workspace already large enough, src/scheduler/prefill.cc:121-124) is
// used instead: the wrapper pre-sizes the six workspace tensors with ordinary host memory, which
// is why this translation unit opens the class's private section.  No reference code is changed.
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include <torch/torch.h>

#define private public
#include "sglang/scheduler/prefill.h"
#undef private
#include "sglang/core/req.h"
#include "sglang/kernels/radix.h"
#include "sglang/kernels/token_pool.h"
#include "sglang/kvcache/cache_manager.h"
#include "sglang/kvcache/radix_tree.h"
#include "sglang/scheduler/decode.h"

namespace sglang {

void write_token_pool(const torch::Tensor& token_pool, const torch::Tensor& req_indices,
                      const torch::Tensor& positions, const torch::Tensor& tokens) {
    TORCH_CHECK(token_pool.dim() == 2 && token_pool.scalar_type() == torch::kInt32, "token_pool must be int32 [rows, cols]");
    const int64_t rows = token_pool.size(0), cols = token_pool.size(1), stride = token_pool.stride(0);
    auto r = req_indices.contiguous(), p = positions.contiguous(), t = tokens.contiguous();
    int32_t* base = token_pool.data_ptr<int32_t>();
    for (int64_t i = 0; i < r.numel(); ++i) {
        const int64_t rr = r.data_ptr<int32_t>()[i], pp = p.data_ptr<int32_t>()[i];
        if (rr < 0 || rr >= rows || pp < 0 || pp >= cols) continue;
        base[rr * stride + pp] = t.data_ptr<int32_t>()[i];
    }
}

torch::Tensor gather_int32_2d(const torch::Tensor& table, const torch::Tensor& req_indices,
                              const torch::Tensor& positions) {
    const int64_t rows = table.size(0), cols = table.size(1), stride = table.stride(0);
    auto r = req_indices.contiguous(), p = positions.contiguous();
    auto out = torch::empty({r.numel()}, torch::kInt32);
    const int32_t* base = table.data_ptr<int32_t>();
    for (int64_t i = 0; i < r.numel(); ++i) {
        const int64_t rr = r.data_ptr<int32_t>()[i], pp = p.data_ptr<int32_t>()[i];
        out.data_ptr<int32_t>()[i] = (rr >= 0 && rr < rows && pp >= 0 && pp < cols) ? base[rr * stride + pp] : 0;
    }
    return out;
}

}  // namespace sglang

namespace {

using namespace sglang;

torch::Tensor ids_tensor(const int32_t* ids, int64_t n) {
    auto t = torch::empty({n}, torch::kInt32);
    if (n > 0) std::memcpy(t.data_ptr<int32_t>(), ids, sizeof(int32_t) * static_cast<size_t>(n));
    return t;
}

thread_local std::string g_err;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

struct HostScheduler {
    int page_size, max_running_req, max_extend_tokens, cols;
    torch::Tensor page_table;
    TableManager table_manager;
    CacheManager cache_manager;
    DecodeManager decode_manager;
    PrefillManager prefill_manager;
    std::shared_ptr<Batch> batch;  // the batch between next_batch and finish_batch

    HostScheduler(int num_pages, int page_size_, int max_running_req_, int max_seq_len, int max_extend_tokens_)
        : page_size(page_size_),
          max_running_req(max_running_req_),
          max_extend_tokens(max_extend_tokens_),
          cols((max_seq_len + 31) / 32 * 32),
          // Engine allocates [max_running_req + 1, align_up(max_seq_len, 32)] int32 (src/engine/engine.cc:452-459)
          page_table(torch::zeros({max_running_req_ + 1, cols}, torch::kInt32)),
          table_manager(max_running_req_, page_table),
          cache_manager(num_pages, page_size_, page_table, "radix"),
          decode_manager(page_size_),
          prefill_manager(cache_manager, table_manager, decode_manager) {
        const int64_t cap = static_cast<int64_t>(num_pages + 1) * page_size_;
        auto mk = [&] { return torch::empty({cap}, torch::kInt32); };
        cache_manager.page_write_table_idx_host_ = mk();
        cache_manager.page_write_positions_host_ = mk();
        cache_manager.page_write_tokens_host_ = mk();
        cache_manager.page_write_table_idx_device_ = mk();
        cache_manager.page_write_positions_device_ = mk();
        cache_manager.page_write_tokens_device_ = mk();
    }
};

struct RadixBox {
    RadixPrefixCache cache;
    std::vector<std::shared_ptr<BaseCacheHandle>> handles;
    explicit RadixBox(int page_size) : cache(page_size) {}
};

}  // namespace

extern "C" {

const char* ref_last_error(void) { return g_err.c_str(); }

// ---- the scheduler's integer side ------------------------------------------------------------

void* ref_sched_create(int num_pages, int page_size, int max_running_req, int max_seq_len, int max_extend_tokens) {
    void* out = nullptr;
    guarded([&] { out = new HostScheduler(num_pages, page_size, max_running_req, max_seq_len, max_extend_tokens); });
    return out;
}

void ref_sched_destroy(void* h) { delete static_cast<HostScheduler*>(h); }

// Scheduler::submit (src/scheduler/scheduler.cc:204-227) without the length clamp's logging.
int ref_sched_submit(void* h, uint64_t uid, const int32_t* ids, int n, int max_new_tokens) {
    auto* s = static_cast<HostScheduler*>(h);
    return guarded([&] {
        GenerateRequest r;
        r.uid = uid;
        r.input_ids = ids_tensor(ids, n);
        r.sampling_params.max_new_tokens = max_new_tokens;
        r.sampling_params.ignore_eos = true;
        s->prefill_manager.add_one_req(std::move(r));
    });
}

// schedule_next_batch (prefill first, else decode; no decode bursts) followed by prepare_batch's
// CacheManager::allocate_paged.  Writes one entry per request; returns the request count, 0 when
// idle, -1 on error.  phase: 0 prefill, 1 decode.
int ref_sched_next_batch(void* h, int* phase, int cap, uint64_t* uids, int32_t* table_idx, int32_t* cached_len,
                         int32_t* device_len, int32_t* chunked, int32_t* write_pos) {
    auto* s = static_cast<HostScheduler*>(h);
    int count = 0;
    int rc = guarded([&] {
        TORCH_CHECK(!s->batch, "ref_sched_next_batch: the previous batch was not finished");
        auto b = s->prefill_manager.schedule_next_batch(s->max_extend_tokens);
        if (!b) b = s->decode_manager.schedule_next_batch();
        if (!b) return;
        s->cache_manager.allocate_paged(b->reqs);
        TORCH_CHECK(static_cast<int>(b->reqs.size()) <= cap, "ref_sched_next_batch: output arrays too small");
        for (size_t i = 0; i < b->reqs.size(); ++i) {
            const auto& r = b->reqs[i];
            uids[i] = r->req_id;
            table_idx[i] = r->table_idx;
            cached_len[i] = r->cached_len;
            device_len[i] = r->device_len();
            chunked[i] = r->is_chunked_prefill ? 1 : 0;
            write_pos[i] = r->can_decode() ? r->device_len() : -1;  // scheduler.cc:321-325
        }
        *phase = b->is_decode() ? 1 : 0;
        count = static_cast<int>(b->reqs.size());
        s->batch = b;
    });
    return rc ? -1 : count;
}

// What follows the forward pass: Engine::forward_batch's complete_one for every request
// (src/engine/engine.cc:516-519), the token write-back (scheduler.cc:374-377), filter_reqs (:388)
// and process_forward_output (:424-470).  finished[i] is set for requests that ended.
int ref_sched_finish_batch(void* h, const int32_t* next_tokens, int n, int32_t* finished) {
    auto* s = static_cast<HostScheduler*>(h);
    return guarded([&] {
        TORCH_CHECK(s->batch && static_cast<int>(s->batch->reqs.size()) == n, "ref_sched_finish_batch: no batch of that size");
        auto b = s->batch;
        s->batch.reset();
        std::vector<int32_t> rows(n), pos(n);
        for (int i = 0; i < n; ++i) {
            rows[i] = b->reqs[i]->table_idx;
            pos[i] = b->reqs[i]->can_decode() ? b->reqs[i]->device_len() : -1;
        }
        for (auto& r : b->reqs) r->complete_one();
        write_token_pool(s->table_manager.token_pool(), ids_tensor(rows.data(), n), ids_tensor(pos.data(), n),
                         ids_tensor(next_tokens, n));
        s->decode_manager.filter_reqs(b->reqs);
        CacheManager::LazyFreeRegion lazy_free(s->cache_manager);
        for (int i = 0; i < n; ++i) {
            auto& req = b->reqs[i];
            finished[i] = 0;
            if (req->is_chunked_prefill) continue;
            req->append_host_token(next_tokens[i]);
            const bool fin = !req->can_decode();
            if (fin) {
                s->decode_manager.remove_req(req);
                s->table_manager.free(req->table_idx);           // Scheduler::free_req_resources
                s->cache_manager.cache_req(req, /*finished=*/true);
                finished[i] = 1;
            } else if (b->is_prefill()) {
                s->cache_manager.cache_req(req, /*finished=*/false);
            }
        }
    });
}

const int32_t* ref_sched_page_table(void* h, int* rows, int* cols) {
    auto* s = static_cast<HostScheduler*>(h);
    *rows = static_cast<int>(s->page_table.size(0));
    *cols = static_cast<int>(s->page_table.size(1));
    return s->page_table.data_ptr<int32_t>();
}

const int32_t* ref_sched_token_pool(void* h) {
    return static_cast<HostScheduler*>(h)->table_manager.token_pool().data_ptr<int32_t>();
}

int ref_sched_sizes(void* h, int64_t* evictable, int64_t* protected_size, int* available_tokens, int* free_rows,
                    int* inflight_tokens, int* pending) {
    auto* s = static_cast<HostScheduler*>(h);
    return guarded([&] {
        auto info = s->cache_manager.prefix_cache_->size_info();
        *evictable = info.evictable_size;
        *protected_size = info.protected_size;
        *available_tokens = s->cache_manager.available_size();
        *free_rows = s->table_manager.available_size();
        *inflight_tokens = s->decode_manager.inflight_tokens();
        *pending = static_cast<int>(s->prefill_manager.pending_size());
        // Pages held by requests in flight are in neither the tree nor the free list, so the
        // reference's check only holds when nothing is running.
        if (!s->decode_manager.runnable() && !s->prefill_manager.runnable()) s->cache_manager.check_integrity();
    });
}

// ---- RadixPrefixCache -----------------------------------------------------------------------------

void* ref_radix_create(int page_size) { return new RadixBox(page_size); }
void ref_radix_destroy(void* h) { delete static_cast<RadixBox*>(h); }

// Returns the length already cached before the insertion; -1 on error.
int64_t ref_radix_insert(void* h, const int32_t* ids, const int32_t* indices, int n, int64_t* handle_len, int* handle_id) {
    auto* b = static_cast<RadixBox*>(h);
    int64_t out = -1;
    guarded([&] {
        auto r = b->cache.insert_prefix(ids_tensor(ids, n), ids_tensor(indices, n));
        b->handles.push_back(r.handle);
        *handle_len = r.handle->cached_len;
        *handle_id = static_cast<int>(b->handles.size()) - 1;
        out = r.cached_len;
    });
    return out;
}

// Returns the matched length and copies the matched indices; -1 on error.
int64_t ref_radix_match(void* h, const int32_t* ids, int n, int* handle_id, int32_t* matched, int cap) {
    auto* b = static_cast<RadixBox*>(h);
    int64_t out = -1;
    guarded([&] {
        auto r = b->cache.match_prefix(ids_tensor(ids, n));
        b->handles.push_back(r.handle);
        *handle_id = static_cast<int>(b->handles.size()) - 1;
        auto idx = r.handle->get_matched_indices().contiguous();
        TORCH_CHECK(idx.numel() <= cap, "ref_radix_match: output too small");
        TORCH_CHECK(idx.numel() == r.handle->cached_len, "matched indices and cached_len disagree");
        if (idx.numel() > 0) std::memcpy(matched, idx.data_ptr<int32_t>(), sizeof(int32_t) * idx.numel());
        out = r.handle->cached_len;
    });
    return out;
}

int ref_radix_lock(void* h, int handle_id, int unlock) {
    auto* b = static_cast<RadixBox*>(h);
    return guarded([&] { b->cache.lock_handle(b->handles.at(handle_id), unlock != 0); });
}

// Returns the number of evicted slots copied to `out`; -1 on error (c10::Error of the reference).
int64_t ref_radix_evict(void* h, int64_t size, int32_t* out, int cap) {
    auto* b = static_cast<RadixBox*>(h);
    int64_t n = -1;
    guarded([&] {
        auto ev = b->cache.evict(size).contiguous();
        TORCH_CHECK(ev.numel() <= cap, "ref_radix_evict: output too small");
        if (ev.numel() > 0) std::memcpy(out, ev.data_ptr<int32_t>(), sizeof(int32_t) * ev.numel());
        n = ev.numel();
    });
    return n;
}

void ref_radix_size(void* h, int64_t* evictable, int64_t* protected_size) {
    auto info = static_cast<RadixBox*>(h)->cache.size_info();
    *evictable = info.evictable_size;
    *protected_size = info.protected_size;
}

// ---- small pieces ----------------------------------------------------------------------------------

int64_t ref_fast_compare_key(const int32_t* a, int na, const int32_t* b, int nb) {
    int64_t out = -1;
    guarded([&] { out = fast_compare_key(ids_tensor(a, na), ids_tensor(b, nb)); });
    return out;
}

int64_t ref_key_fn(int page_size, const int32_t* ids, int n) {
    int64_t out = 0;
    guarded([&] { out = get_key_fn(page_size)(ids_tensor(ids, n)); });
    return out;
}

// RadixTreeNode::split_at on a child of a fresh root; writes the lengths, keys and values of the
// new prefix node and of the shortened node, plus the prefix node's ref_count.
int ref_node_split(const int32_t* key, const int32_t* value, int n, int pos, int ref_count, int32_t* prefix_key,
                   int32_t* prefix_value, int32_t* suffix_key, int32_t* suffix_value, int* prefix_ref_count,
                   int* parent_ok) {
    return guarded([&] {
        auto key_fn = get_key_fn(1);
        auto root = std::make_unique<RadixTreeNode>(key_fn);
        root->ref_count = 1;
        auto child = std::make_unique<RadixTreeNode>(key_fn);
        child->set_key_value(ids_tensor(key, n), ids_tensor(value, n));
        child->set_parent(root.get());
        child->ref_count = ref_count;
        std::unique_ptr<RadixTreeNode> fresh(child->split_at(pos));
        TORCH_CHECK(fresh->length() == pos && child->length() == n - pos, "split lengths");
        std::memcpy(prefix_key, fresh->key().contiguous().data_ptr<int32_t>(), sizeof(int32_t) * pos);
        std::memcpy(prefix_value, fresh->value().contiguous().data_ptr<int32_t>(), sizeof(int32_t) * pos);
        std::memcpy(suffix_key, child->key().contiguous().data_ptr<int32_t>(), sizeof(int32_t) * (n - pos));
        std::memcpy(suffix_value, child->value().contiguous().data_ptr<int32_t>(), sizeof(int32_t) * (n - pos));
        *prefix_ref_count = fresh->ref_count;
        *parent_ok = (fresh->parent() == root.get() && child->parent() == fresh.get() && !fresh->is_leaf()) ? 1 : 0;
    });
}

// ---- Req -------------------------------------------------------------------------------------------

void* ref_req_create(const int32_t* ids, int n, int cached_len, int output_len, int chunked, int initialize) {
    Req* r = nullptr;
    guarded([&] {
        r = new Req();
        r->input_ids = ids_tensor(ids, n);
        r->cached_len = cached_len;
        r->output_len = output_len;
        r->is_chunked_prefill = chunked != 0;
        if (initialize) r->initialize_runtime_state();
    });
    return r;
}
void ref_req_destroy(void* h) { delete static_cast<Req*>(h); }
// out: device_len, max_device_len, remain_len, extend_len, can_decode, cached_len, host length
void ref_req_state(void* h, int32_t out[7]) {
    auto* r = static_cast<Req*>(h);
    out[0] = r->device_len();
    out[1] = r->max_device_len();
    out[2] = r->remain_len();
    out[3] = r->extend_len();
    out[4] = r->can_decode() ? 1 : 0;
    out[5] = r->cached_len;
    out[6] = static_cast<int32_t>(r->input_ids.size(0));
}
int ref_req_complete_one(void* h) {
    return guarded([&] { static_cast<Req*>(h)->complete_one(); });
}
int ref_req_append_host(void* h, int32_t token) {
    return guarded([&] {
        auto t = torch::empty({1}, torch::kInt32);
        t.data_ptr<int32_t>()[0] = token;
        static_cast<Req*>(h)->append_host(t);
    });
}

}  // extern "C"
