// Link-time drop-in check: the reference's own Engine, built from the reference's unchanged sources
// with the four adapter translation units of this directory in place of the four FlashInfer-bound
// ones, against the step runner of libb200_token_loop.so on the same weights.
//
// The probe constructs sglang::Engine (src/engine/engine.cc:412-489) with a small dummy model,
// rescales its random weights to the N(0, 0.02) / norm-weights-1 distribution of the test
// configurations, runs Engine::forward_batch for one prefill batch and some decode steps, copies the
// very same weights into a b200_engine and runs the same requests through b200_engine_step.  It
// prints one JSON line with both token sequences; tests/test_adapters_gpu.py compares them.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/torch.h>

#include "b200_token_loop.h"
#include "sglang/core/batch.h"
#include "sglang/core/req.h"
#define private public   // the probe reads the model's parameters, which Engine keeps private
#include "sglang/engine/engine.h"
#undef private
#include "sglang/kernels/token_pool.h"

using namespace sglang;

namespace {

void ok(int status, const char* what) {
    if (status != B200_OK) {
        std::fprintf(stderr, "%s failed: %s\n", what, b200_last_error());
        std::exit(2);
    }
}

std::string join(const std::vector<int>& v) {
    std::string s = "[";
    for (size_t i = 0; i < v.size(); ++i) s += (i ? "," : "") + std::to_string(v[i]);
    return s + "]";
}

}  // namespace

int main(int argc, char** argv) {
    const std::string mode = argc < 2 ? "qwen3" : argv[1];
    const bool qwen3 = mode != "llama";
    const bool graphs = mode == "qwen3-graph";   // decode steps replay CUDA graphs captured by GraphRunner
    const int steps = 6;
    ModelConfig mc{};
    mc.num_layers = 2;
    mc.num_qo_heads = 4;
    mc.num_kv_heads = 2;
    mc.head_dim = 128;
    mc.hidden_size = 256;
    mc.vocab_size = 2048;
    mc.intermediate_size = 512;
    mc.rms_norm_eps = 1e-6f;
    mc.rotary_config.base = qwen3 ? 1e6f : 5e5f;
    mc.rotary_config.max_position = 512;
    mc.rotary_config.rotary_dim = 128;
    mc.rotary_config.head_dim = 128;
    mc.hidden_act = "silu";
    mc.num_experts = 0;
    mc.num_experts_per_tok = 0;
    mc.moe_intermediate_size = 0;
    mc.norm_topk_prob = false;
    mc.tie_word_embeddings = false;
    mc.model_type = qwen3 ? "qwen3" : "llama";
    mc.architectures = {qwen3 ? "Qwen3ForCausalLM" : "LlamaForCausalLM"};

    EngineConfig ec;
    ec.dtype = torch::kBFloat16;
    ec.max_running_req = 4;
    ec.page_size = 1;
    ec.use_dummy_weight = true;
    ec.num_pages_override = 256;
    ec.max_seq_len_override = 128;
    ec.model_config_override = mc;
    if (graphs) {
        ec.enable_cuda_graph = true;
        ec.cuda_graph_batch_sizes = {2, 4};
        ec.cuda_graph_capture_max_seq_len = 128;
    }
    Engine engine(ec);
    c10::cuda::CUDAGuard guard(engine.device());

    // the test configurations' weight distribution: matrices N(0, 0.02), norm weights 1
    torch::NoGradGuard no_grad;
    std::vector<std::pair<std::string, torch::Tensor>> params;
    for (auto& entry : engine.model_runner_.module->named_parameters(/*recurse=*/true)) {
        auto& t = entry.value();
        if (t.dim() == 1) t.fill_(1.0); else t.mul_(0.02);
        params.emplace_back(entry.key(), t);
    }

    // ---- requests: two prompts, page size 1, slots handed out in order ----
    const std::vector<std::vector<int32_t>> prompts = {{5, 17, 300, 9, 1024, 77, 3}, {40, 41, 42, 43, 44, 45, 46, 47, 48, 49, 50, 51}};
    auto page_table = engine.page_table();
    auto token_pool = torch::zeros_like(page_table);
    std::vector<std::shared_ptr<Req>> reqs;
    int next_slot = 0;
    for (size_t i = 0; i < prompts.size(); ++i) {
        auto r = std::make_shared<Req>();
        r->req_id = i + 1;
        r->input_ids = torch::tensor(prompts[i], torch::kInt32);
        r->table_idx = static_cast<int>(ec.max_running_req - 1 - i);
        r->cached_len = 0;
        r->output_len = steps + 2;
        r->sampling_params.ignore_eos = true;
        r->sampling_params.temperature = 0.0f;   // greedy (the default temperature of 1 samples)
        r->initialize_runtime_state();
        for (int p = 0; p < r->max_device_len(); ++p) page_table[r->table_idx][p] = next_slot++;
        token_pool[r->table_idx].slice(0, 0, static_cast<int64_t>(prompts[i].size()))
            .copy_(r->input_ids.to(token_pool.device()));
        reqs.push_back(r);
    }

    // ---- the reference Engine, stepping as Scheduler::prepare_batch + forward do ----
    std::vector<int> ref_tokens;
    auto run_ref = [&](BatchPhase phase) {
        // everything on the engine's stream, as Scheduler::forward orders it (src/scheduler/scheduler.cc:391-412)
        c10::cuda::CUDAStreamGuard stream_guard(engine.stream());
        Batch batch;
        batch.reqs = reqs;
        batch.phase = phase;
        engine.pad_batch(batch);
        std::vector<int32_t> rows, pos;
        for (auto& r : batch.padded_reqs)
            for (int p = r->cached_len; p < r->device_len(); ++p) {
                rows.push_back(r->table_idx);
                pos.push_back(p);
            }
        auto dev = engine.device();
        auto rows_t = torch::tensor(rows, torch::kInt32).to(dev), pos_t = torch::tensor(pos, torch::kInt32).to(dev);
        batch.positions = pos_t;
        batch.out_loc = gather_int32_2d(page_table, rows_t, pos_t);
        batch.input_ids = gather_int32_2d(token_pool, rows_t, pos_t);
        engine.prepare_attention_metadata(batch);
        auto args = engine.prepare_sampling_args(batch);
        std::vector<int32_t> wrow, wpos;
        for (auto& r : batch.reqs) {
            wrow.push_back(r->table_idx);
            wpos.push_back(r->can_decode() ? r->device_len() : -1);
        }
        auto out = engine.forward_batch(batch, args);
        write_token_pool(token_pool, torch::tensor(wrow, torch::kInt32).to(dev), torch::tensor(wpos, torch::kInt32).to(dev),
                         out.next_tokens_gpu);
        out.synchronize();
        for (size_t i = 0; i < reqs.size(); ++i) ref_tokens.push_back(out.next_tokens_cpu[i].item<int>());
    };
    run_ref(BatchPhase::Prefill);
    for (int s = 0; s < steps; ++s) run_ref(BatchPhase::Decode);

    // ---- the step runner on the same weights and requests ----
    b200_model_config m = {};
    m.num_layers = mc.num_layers;
    m.hidden_size = mc.hidden_size;
    m.num_qo_heads = mc.num_qo_heads;
    m.num_kv_heads = mc.num_kv_heads;
    m.head_dim = mc.head_dim;
    m.intermediate_size = mc.intermediate_size;
    m.vocab_size = mc.vocab_size;
    m.rms_norm_eps = mc.rms_norm_eps;
    m.rope_theta = mc.rotary_config.base;
    m.max_position = mc.rotary_config.max_position;
    m.tie_word_embeddings = 0;
    m.qk_norm = qwen3 ? 1 : 0;
    m.fused_residual = qwen3 ? 1 : 0;
    b200_engine_config c = {};
    c.page_size = 1;
    c.num_pages = 256;
    c.max_running_req = ec.max_running_req;
    c.max_seq_len = 128;
    c.max_extend_tokens = 256;
    c.tp_size = 1;
    b200_engine* e = nullptr;
    ok(b200_engine_create(&m, &c, &e), "b200_engine_create");
    auto find = [&](const std::string& suffix) -> torch::Tensor {
        for (auto& kv : params)
            if (kv.first.size() >= suffix.size() && kv.first.compare(kv.first.size() - suffix.size(), suffix.size(), suffix) == 0)
                return kv.second;
        std::fprintf(stderr, "no parameter ending in %s\n", suffix.c_str());
        std::exit(3);
    };
    auto load = [&](const char* name, int layer, const torch::Tensor& t) {
        auto h = t.to(torch::kCPU).contiguous();
        ok(b200_engine_load(e, name, layer, h.data_ptr(), static_cast<int64_t>(h.numel() * h.element_size())), name);
    };
    if (argc > 2) for (auto& kv : params) std::fprintf(stderr, "param %s\n", kv.first.c_str());
    load("embed", 0, find("embed_tokens.weight"));
    load("lm_head", 0, find("lm_head.weight"));
    load("final_norm", 0, find("model.norm.weight"));   // registered names: src/models/qwen3.cc:38-52,69-77
    for (int l = 0; l < mc.num_layers; ++l) {
        const std::string p = "layers_" + std::to_string(l) + ".";
        load("qkv", l, find(p + "self_attn.qkv_proj.weight"));
        load("o", l, find(p + "self_attn.o_proj.weight"));
        load("gate_up", l, find(p + "mlp.gate_up_proj.weight"));
        load("down", l, find(p + "mlp.down_proj.weight"));
        load("input_norm", l, find(p + "input_layernorm.weight"));
        load("post_norm", l, find(p + "post_attention_layernorm.weight"));
        if (qwen3) {
            load("q_norm", l, find(p + "self_attn.q_norm.weight"));
            load("k_norm", l, find(p + "self_attn.k_norm.weight"));
        }
    }
    std::vector<int32_t> rows, pos, val;
    int slot = 0;
    for (size_t i = 0; i < prompts.size(); ++i) {
        const int row = ec.max_running_req - 1 - static_cast<int>(i);
        const int maxlen = static_cast<int>(prompts[i].size()) + steps + 2;
        for (int p = 0; p < maxlen; ++p) {
            rows.push_back(row);
            pos.push_back(p);
            val.push_back(slot++);
        }
    }
    ok(b200_engine_write_table(e, 0, rows.data(), pos.data(), val.data(), static_cast<int64_t>(rows.size())), "page table");
    rows.clear(); pos.clear(); val.clear();
    for (size_t i = 0; i < prompts.size(); ++i)
        for (size_t p = 0; p < prompts[i].size(); ++p) {
            rows.push_back(ec.max_running_req - 1 - static_cast<int>(i));
            pos.push_back(static_cast<int>(p));
            val.push_back(prompts[i][p]);
        }
    ok(b200_engine_write_table(e, 1, rows.data(), pos.data(), val.data(), static_cast<int64_t>(rows.size())), "token pool");
    std::vector<int> own_tokens;
    std::vector<int32_t> table_idx, cached, extend, write_pos, toks(prompts.size());
    for (int s = 0; s <= steps; ++s) {
        table_idx.clear(); cached.clear(); extend.clear(); write_pos.clear();
        for (size_t i = 0; i < prompts.size(); ++i) {
            const int len = static_cast<int>(prompts[i].size());
            table_idx.push_back(ec.max_running_req - 1 - static_cast<int>(i));
            cached.push_back(s == 0 ? 0 : len + s - 1);
            extend.push_back(s == 0 ? len : 1);
            write_pos.push_back(len + s);
        }
        b200_step st = {};
        st.phase = s == 0 ? B200_PHASE_PREFILL : B200_PHASE_DECODE;
        st.num_reqs = st.num_padded_reqs = static_cast<int>(prompts.size());
        st.table_idx = table_idx.data();
        st.cached_lens = cached.data();
        st.extend_lens = extend.data();
        st.write_pos = write_pos.data();
        ok(b200_engine_step(e, &st, toks.data()), "b200_engine_step");
        ok(b200_engine_synchronize(e), "b200_engine_synchronize");
        for (int t : toks) own_tokens.push_back(t);
    }
    b200_engine_destroy(e);
    std::printf("{\"model\": \"%s\", \"reference_engine_with_adapters\": %s, \"b200_engine_step\": %s}\n",
                mode.c_str(), join(ref_tokens).c_str(), join(own_tokens).c_str());
    return 0;
}
