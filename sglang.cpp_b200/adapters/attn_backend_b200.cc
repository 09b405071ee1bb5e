// sglang::FlashInferBackend and FlashInferAttnMetadata (include/sglang/attention/flashinfer_backend.h:16-37,
// include/sglang/attention/backend.h:24-41) on the C ABI.  Replaces src/attention/flashinfer_backend.cu.
//
// The class keeps its name and declaration (Engine constructs it by name, src/engine/engine.cc:451-455)
// but none of FlashInfer's host-side planning: the kernels behind b200_attention_decode / _prefill read
// page_table rows directly and split the keys on the device, so
//   * prepare_metadata uploads, per padded request, the table row and device_len (and the query
//     offsets of a prefill batch) — no CSR of slots is built (`indices` stays empty);
//   * a decode step is capturable as it stands: init_capture_graph allocates fixed buffers for the
//     largest batch, prepare_for_capture points the metadata at them, prepare_for_replay copies the
//     step's rows and lengths into them (what the reference does for its plan,
//     src/attention/flashinfer_backend.cu:193-352).
// The fields Scheduler and select_lm_head_input read (src/scheduler/scheduler.cc:171-179,
// src/models/utils.cc:14) are filled: indptr (prefill: query offsets; decode: key offsets),
// paged_kv_indptr, paged_kv_last_page_len.
#include "sglang/attention/flashinfer_backend.h"

#include <cmath>

#include <c10/cuda/CUDAGuard.h>

#include "adapter_common.h"
#include "sglang/core/batch.h"
#include "sglang/core/context.h"
#include "sglang/kvcache/base.h"

namespace sglang {

using b200_adapters::check;
using b200_adapters::current_stream;
using b200_adapters::require_bf16;

namespace {

// What the kernels need beyond the reference's metadata fields; kept behind decode_plan_state.
struct B200StepTables {
    torch::Tensor table_idx;   // int32 [bs] device: page-table row per padded request
    torch::Tensor seq_lens;    // int32 [bs] device: device_len per padded request
    int max_extend = 1;
};

torch::Tensor pinned_i32(const std::vector<int32_t>& v) {
    auto t = torch::empty({static_cast<int64_t>(v.size())},
                          torch::TensorOptions().dtype(torch::kInt32).device(torch::kCPU).pinned_memory(true));
    std::memcpy(t.data_ptr<int32_t>(), v.data(), v.size() * sizeof(int32_t));
    return t;
}

B200StepTables* tables_of(const FlashInferAttnMetadata& m) {
    auto* t = static_cast<B200StepTables*>(m.decode_plan_state.get());
    TORCH_CHECK(t != nullptr, "attention metadata was not prepared by this backend");
    return t;
}

}  // namespace

torch::Tensor FlashInferAttnMetadata::get_last_indices(int bs) const {
    return indptr.slice(0, 1, bs + 1) - 1;
}

FlashInferBackend::FlashInferBackend(std::shared_ptr<BaseKVCachePool> kv_cache, int num_qo_heads, int num_kv_heads,
                                     int head_dim)
    : kv_cache_(kv_cache), num_qo_heads_(num_qo_heads), num_kv_heads_(num_kv_heads), head_dim_(head_dim) {
    TORCH_CHECK(head_dim == 128, "the sm_100a attention kernels take head_dim 128");
    // split-KV scratch of the decode kernel for up to 1024 requests (partials are written before
    // they are read, so it needs no initialisation)
    const int64_t bytes = b200_attention_decode_workspace_bytes(1024, num_qo_heads, num_kv_heads, head_dim);
    TORCH_CHECK(bytes > 0, "unsupported head configuration for decode attention: ", num_qo_heads, " / ", num_kv_heads);
    float_workspace_ = torch::zeros({bytes}, torch::TensorOptions().dtype(torch::kByte).device(kv_cache_->device()));
}

void FlashInferBackend::prepare_metadata(Batch& batch) {
    c10::cuda::OptionalCUDAGuard device_guard(kv_cache_->device());
    auto metadata = std::make_shared<FlashInferAttnMetadata>();
    metadata->is_prefill = batch.is_prefill();
    const int bs = static_cast<int>(batch.padded_reqs.size());
    auto device = kv_cache_->device();
    auto tables = std::make_shared<B200StepTables>();

    std::vector<int32_t> rows(bs), lens(bs);
    metadata->qo_indptr_host = {0};
    metadata->kv_indptr_host = {0};
    for (int i = 0; i < bs; ++i) {
        const auto& req = batch.padded_reqs[i];
        rows[i] = req->table_idx;
        lens[i] = req->device_len();
        metadata->seq_lens.push_back(req->device_len());
        metadata->cached_lens.push_back(req->cached_len);
        const int ext = metadata->is_prefill ? std::max(1, req->extend_len()) : 1;
        tables->max_extend = std::max(tables->max_extend, ext);
        metadata->qo_indptr_host.push_back(metadata->qo_indptr_host.back() + ext);
        metadata->kv_indptr_host.push_back(metadata->kv_indptr_host.back() + req->device_len());
    }
    metadata->last_page_len_host.assign(bs, 1);
    tables->table_idx = pinned_i32(rows).to(device, /*non_blocking=*/true);
    tables->seq_lens = pinned_i32(lens).to(device, /*non_blocking=*/true);
    auto qo = pinned_i32(metadata->qo_indptr_host).to(device, /*non_blocking=*/true);
    auto kv = pinned_i32(metadata->kv_indptr_host).to(device, /*non_blocking=*/true);
    metadata->kv_indptr_host_tensor = pinned_i32(metadata->kv_indptr_host);
    metadata->indptr = metadata->is_prefill ? qo : kv;
    metadata->paged_kv_indptr = kv;
    metadata->indices = torch::empty({0}, torch::TensorOptions().dtype(torch::kInt32).device(device));
    metadata->paged_kv_last_page_len = torch::ones({bs}, torch::TensorOptions().dtype(torch::kInt32).device(device));
    metadata->decode_plan_state = tables;
    metadata->initialized = true;
    metadata->use_capture_buffers = false;
    if (metadata->is_prefill) {
        // the prefill kernel also wants the query offsets on the device: keep them next to the tables
        tables->seq_lens = tables->seq_lens;   // (device_len per request; indptr holds the offsets)
    }
    batch.attn_metadata = metadata;
}

torch::Tensor FlashInferBackend::forward(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                                         int layer_id, Batch& batch) {
    c10::cuda::OptionalCUDAGuard device_guard(kv_cache_->device());
    auto meta = std::dynamic_pointer_cast<FlashInferAttnMetadata>(batch.attn_metadata);
    TORCH_CHECK(meta, "FlashInferBackend requires FlashInferAttnMetadata");
    auto* tables = tables_of(*meta);

    auto k_3d = k.dim() == 2 ? k.view({-1, num_kv_heads_, head_dim_}) : k;
    auto v_3d = v.dim() == 2 ? v.view({-1, num_kv_heads_, head_dim_}) : v;
    kv_cache_->store_kv(k_3d, v_3d, batch.out_loc, layer_id);

    auto q_view = q.view({-1, num_qo_heads_, head_dim_});
    require_bf16(q_view, "q");
    TORCH_CHECK(q_view.stride(2) == 1, "q must have a contiguous last dimension");
    auto o = torch::empty({q_view.size(0), static_cast<int64_t>(num_qo_heads_) * head_dim_}, q.options());

    auto k_cache = kv_cache_->k_cache(layer_id).view({-1, num_kv_heads_, head_dim_});
    auto v_cache = kv_cache_->v_cache(layer_id).view({-1, num_kv_heads_, head_dim_});
    require_bf16(k_cache, "the KV cache");
    auto ctx = get_global_ctx();
    auto page_table = ctx->page_table;
    TORCH_CHECK(page_table.scalar_type() == torch::kInt32 && page_table.stride(1) == 1, "page_table must be int32 rows");
    const int bs = static_cast<int>(batch.padded_reqs.size());
    const float sm_scale = 1.0f / std::sqrt(static_cast<float>(head_dim_));

    if (!meta->is_prefill) {
        TORCH_CHECK(q_view.size(0) == bs, "a decode batch runs one query row per request");
        check(b200_attention_decode(o.data_ptr(), q_view.data_ptr(), q_view.stride(0), q_view.stride(1),
                                    k_cache.data_ptr(), v_cache.data_ptr(), k_cache.size(0),
                                    page_table.data_ptr<int32_t>(), page_table.stride(0),
                                    tables->table_idx.data_ptr<int32_t>(), tables->seq_lens.data_ptr<int32_t>(), bs,
                                    num_qo_heads_, num_kv_heads_, head_dim_, ctx->page_size, sm_scale,
                                    float_workspace_.data_ptr(), float_workspace_.numel(), current_stream()),
              "b200_attention_decode");
    } else {
        check(b200_attention_prefill(o.data_ptr(), q_view.data_ptr(), q_view.stride(0), q_view.stride(1),
                                     k_cache.data_ptr(), v_cache.data_ptr(), k_cache.size(0),
                                     page_table.data_ptr<int32_t>(), page_table.stride(0),
                                     tables->table_idx.data_ptr<int32_t>(), tables->seq_lens.data_ptr<int32_t>(),
                                     meta->indptr.data_ptr<int32_t>(), bs, tables->max_extend, num_qo_heads_,
                                     num_kv_heads_, head_dim_, ctx->page_size, sm_scale, current_stream()),
              "b200_attention_prefill");
    }
    return o;
}

void FlashInferBackend::init_capture_graph(int max_seq_len, const std::vector<int>& bs_list) {
    c10::cuda::OptionalCUDAGuard device_guard(kv_cache_->device());
    decode_capture_.reset();
    if (bs_list.empty()) return;
    decode_capture_ = std::make_unique<DecodeCaptureData>();
    decode_capture_->max_seq_len = max_seq_len;
    decode_capture_->batch_sizes = bs_list;
    decode_capture_->max_batch_size = *std::max_element(bs_list.begin(), bs_list.end());
    auto dev = torch::TensorOptions().dtype(torch::kInt32).device(kv_cache_->device());
    const int64_t n = decode_capture_->max_batch_size;
    decode_capture_->kv_indptr_host = torch::zeros({n + 1}, torch::TensorOptions().dtype(torch::kInt32).pinned_memory(true));
    decode_capture_->kv_indptr_device = torch::zeros({n + 1}, dev);
    decode_capture_->indices = torch::zeros({2 * n}, dev);   // fixed buffers: [table rows | device lengths]
    decode_capture_->last_page_len = torch::ones({n}, dev);
}

void FlashInferBackend::prepare_for_capture(Batch& batch) {
    c10::cuda::OptionalCUDAGuard device_guard(kv_cache_->device());
    TORCH_CHECK(batch.is_decode(), "FlashInfer capture only supports decode batches");
    TORCH_CHECK(decode_capture_, "Decode capture state is not initialized");
    const int bs = batch.padded_size();
    const int64_t n = decode_capture_->max_batch_size;
    auto metadata = std::make_shared<FlashInferAttnMetadata>();
    metadata->is_prefill = false;
    metadata->use_capture_buffers = true;
    metadata->initialized = true;
    metadata->indptr = decode_capture_->kv_indptr_device.slice(0, 0, bs + 1);
    metadata->paged_kv_indptr = metadata->indptr;
    metadata->indices = torch::empty({0}, decode_capture_->indices.options());
    metadata->paged_kv_last_page_len = decode_capture_->last_page_len.slice(0, 0, bs);
    metadata->kv_indptr_host_tensor = decode_capture_->kv_indptr_host.slice(0, 0, bs + 1);
    metadata->last_page_len_host.assign(bs, 1);
    auto tables = std::make_shared<B200StepTables>();
    tables->table_idx = decode_capture_->indices.slice(0, 0, bs);
    tables->seq_lens = decode_capture_->indices.slice(0, n, n + bs);
    // the capture runs on the dummy request: its row, one key each
    tables->table_idx.fill_(batch.padded_reqs.front()->table_idx);
    tables->seq_lens.fill_(1);
    metadata->decode_plan_state = tables;
    decode_capture_->metadata[bs] = metadata;
    batch.attn_metadata = metadata;
}

void FlashInferBackend::prepare_for_replay(Batch& batch) {
    c10::cuda::OptionalCUDAGuard device_guard(kv_cache_->device());
    TORCH_CHECK(batch.is_decode(), "FlashInfer replay only supports decode batches");
    auto metadata = std::dynamic_pointer_cast<FlashInferAttnMetadata>(batch.attn_metadata);
    TORCH_CHECK(metadata, "FlashInfer replay requires FlashInferAttnMetadata");
    TORCH_CHECK(decode_capture_, "Decode capture state is not initialized");
    const int bs = batch.padded_size();
    auto it = decode_capture_->metadata.find(bs);
    TORCH_CHECK(it != decode_capture_->metadata.end(), "No decode capture metadata for batch size ", bs);
    auto capture = it->second;
    auto* src = tables_of(*metadata);
    auto* dst = tables_of(*capture);
    dst->table_idx.copy_(src->table_idx, /*non_blocking=*/true);
    dst->seq_lens.copy_(src->seq_lens, /*non_blocking=*/true);
    capture->indptr.copy_(metadata->indptr, /*non_blocking=*/true);
    capture->seq_lens = metadata->seq_lens;
    capture->cached_lens = metadata->cached_lens;
    batch.attn_metadata = capture;
}

}  // namespace sglang
