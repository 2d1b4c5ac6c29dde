// Times tianyuxbear/zedinfer's own NVIDIA path on a Qwen2 shape with random weights, the way its profiler and its
// serving loop drive it (src/zedinfer/profiler.cpp:119-162, src/zedinfer/serving_loop.cpp:206-289,
// src/zedinfer/scheduler.cpp:765-790): its unmodified transformer_forward over its PagedForwardContext, BlockPool
// and BlockAllocator, its CUDA kernels, cuBLASLt and FlashInfer wrappers, and its ArgmaxSampler for the token of
// every request.  Nothing of zedinfer_b200 is linked or called here; this file only builds the model from a list of
// sizes, fills the weights with random numbers and runs the reference's calls in the reference's order.
//
//   ref_bench L H I V nh nkv hd theta eps block_size  <jobs...>
//   jobs:  prefill:<tokens>:<rounds>:<warmup>      one prompt of that many tokens, alone
//          decode:<batch>:<context0>:<steps>:<warmup>   `batch` requests that hold `context0` tokens each,
//                                                 then warmup + steps decode steps of the whole batch
// Prints one line per job: "prefill tokens ms_median ms_min ms_max" / "decode batch context0 steps ms_per_step ms_total".
#include "backend/core/context/context.hpp"
#include "backend/kvcache/block_pool.hpp"
#include "backend/tensor/tensor.hpp"
#include "frontend/models/decode_scratch.hpp"
#include "frontend/models/forward_config.hpp"
#include "frontend/models/paged_forward_context.hpp"
#include "frontend/models/qwen2.hpp"
#include "frontend/sampler/sampler.hpp"
#include "zedinfer/activation.hpp"
#include "zedinfer/batch_context.hpp"
#include "zedinfer/request.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

using namespace zedinfer;
using clk = std::chrono::high_resolution_clock;

static uint64_t g_state = 0x9E3779B97F4A7C15ull;
static inline uint32_t next_u32() {
    g_state ^= g_state << 13; g_state ^= g_state >> 7; g_state ^= g_state << 17;
    return (uint32_t)(g_state >> 32);
}
// sum of four uniforms, centred: close enough to a normal for timing purposes; returned as bfloat16 bits
static inline uint16_t random_bf16(float std_, float mean) {
    float s = 0.0f;
    for (int i = 0; i < 4; ++i) s += (float)(next_u32() >> 8) * (1.0f / 16777216.0f);
    const float x = mean + std_ * (s - 2.0f) * 1.7320508f;
    uint32_t u;
    memcpy(&u, &x, 4);
    u += 0x7FFF + ((u >> 16) & 1);
    return (uint16_t)(u >> 16);
}

static tensor_t device_tensor(const std::vector<size_t>& shape, float std_, float mean) {
    size_t n = 1;
    for (auto s : shape) n *= s;
    std::vector<uint16_t> host(n);
    for (auto& v : host) v = random_bf16(std_, mean);
    auto t = Tensor::create(shape, ZEDINFER_DTYPE_BF16, ZEDINFER_DEVICE_NVIDIA, 0);
    t->load(host.data());
    return t;
}

static double ms_since(clk::time_point t0) { return std::chrono::duration<double, std::milli>(clk::now() - t0).count(); }

static std::vector<int> random_ids(size_t n, int vocab) {       // as the reference's profiler: ids in [100, vocab - 100]
    std::vector<int> v(n);
    for (auto& t : v) t = 100 + (int)(next_u32() % (uint32_t)(vocab - 200));
    return v;
}

int main(int argc, char** argv) {
    if (argc < 12) { std::cerr << "usage: ref_bench L H I V nh nkv hd theta eps block_size jobs...\n"; return 2; }
    model::ModelConfig base;
    base.num_hidden_layers = std::atoi(argv[1]);
    base.hidden_size = std::atoi(argv[2]);
    base.intermediate_size = std::atoi(argv[3]);
    base.vocab_size = std::atoi(argv[4]);
    base.num_attention_heads = std::atoi(argv[5]);
    base.num_key_value_heads = std::atoi(argv[6]);
    base.head_dim = std::atoi(argv[7]);
    base.rope_theta = std::atof(argv[8]);
    base.rms_norm_eps = std::atof(argv[9]);
    const int block_size = std::atoi(argv[10]);
    base.tie_word_embeddings = false;
    base.max_position_embeddings = 32768;
    base.model_type = "qwen2";
    base.torch_dtype = "bfloat16";
    const size_t L = base.num_hidden_layers, H = base.hidden_size, I = base.intermediate_size, V = base.vocab_size;
    const size_t qd = base.num_attention_heads * base.head_dim, kd = base.num_key_value_heads * base.head_dim;

    core::context().setDevice(ZEDINFER_DEVICE_NVIDIA, 0);
    auto weights = std::make_unique<model::ModelWeights>();
    weights->add_tensor("embed_tokens.weight", device_tensor({V, H}, 0.02f, 0.0f));
    weights->add_tensor("lm_head.weight", device_tensor({V, H}, 0.02f, 0.0f));
    weights->add_tensor("norm.weight", device_tensor({H}, 0.01f, 1.0f));
    for (size_t l = 0; l < L; ++l) {
        const std::string p = "layers." + std::to_string(l) + ".";
        weights->add_tensor(p + "input_layernorm.weight", device_tensor({H}, 0.01f, 1.0f));
        weights->add_tensor(p + "post_attention_layernorm.weight", device_tensor({H}, 0.01f, 1.0f));
        weights->add_tensor(p + "self_attn.q_proj.weight", device_tensor({qd, H}, 0.02f, 0.0f));
        weights->add_tensor(p + "self_attn.q_proj.bias", device_tensor({qd}, 0.02f, 0.0f));
        weights->add_tensor(p + "self_attn.k_proj.weight", device_tensor({kd, H}, 0.02f, 0.0f));
        weights->add_tensor(p + "self_attn.k_proj.bias", device_tensor({kd}, 0.02f, 0.0f));
        weights->add_tensor(p + "self_attn.v_proj.weight", device_tensor({kd, H}, 0.02f, 0.0f));
        weights->add_tensor(p + "self_attn.v_proj.bias", device_tensor({kd}, 0.02f, 0.0f));
        weights->add_tensor(p + "self_attn.o_proj.weight", device_tensor({H, qd}, 0.02f, 0.0f));
        weights->add_tensor(p + "mlp.gate_proj.weight", device_tensor({I, H}, 0.02f, 0.0f));
        weights->add_tensor(p + "mlp.up_proj.weight", device_tensor({I, H}, 0.02f, 0.0f));
        weights->add_tensor(p + "mlp.down_proj.weight", device_tensor({H, I}, 0.02f, 0.0f));
    }
    model::Qwen2Config qcfg(base);
    qcfg.sliding_window = 4096; qcfg.max_window_layers = 21; qcfg.use_sliding_window = false;
    model::Qwen2Model qwen(qcfg, std::move(weights));
    const auto fcfg = qwen.forward_config();
    ExecutorConfig exec(ZEDINFER_DEVICE_NVIDIA, 0, ZEDINFER_DTYPE_BF16, 32768);
    auto scratch = model::DecodeScratch::create(qwen.config(), fcfg, exec);
    sampler::ArgmaxSampler argmax(exec);
    auto* api = core::context().runtime().api();

    // the pool: enough pages for the largest job (every layer has page ids of its own in the reference)
    size_t most_tokens = 0;
    std::vector<std::vector<std::string>> jobs;
    for (int a = 11; a < argc; ++a) {
        std::vector<std::string> f;
        std::stringstream ss(argv[a]);
        std::string item;
        while (std::getline(ss, item, ':')) f.push_back(item);
        jobs.push_back(f);
        if (f[0] == "prefill") most_tokens = std::max(most_tokens, (size_t)std::atoi(f[1].c_str()) + 64);
        if (f[0] == "decode")
            most_tokens = std::max(most_tokens, (size_t)std::atoi(f[1].c_str())
                                                    * ((size_t)std::atoi(f[2].c_str()) + std::atoi(f[3].c_str()) + std::atoi(f[4].c_str()) + 2 * block_size));
    }
    kvcache::BlockConfig bc;
    bc.block_size = block_size; bc.num_kv_heads = (int)base.num_key_value_heads; bc.head_dim = (int)base.head_dim;
    bc.dtype = ZEDINFER_DTYPE_BF16;
    const int blocks = (int)((most_tokens / block_size + 64) * L);
    kvcache::BlockPool pool(bc, blocks, ZEDINFER_DEVICE_NVIDIA, 0);
    kvcache::BlockAllocator alloc(pool, (int)L);

    for (const auto& f : jobs) {
        if (f[0] == "prefill") {
            const int n = std::atoi(f[1].c_str()), rounds = std::atoi(f[2].c_str()), warm = std::atoi(f[3].c_str());
            std::vector<double> ms;
            for (int r = 0; r < warm + rounds; ++r) {
                auto table = alloc.allocate_sequence(n + 1);
                auto ids = random_ids(n, (int)V);
                alloc.ensure_blocks(table, n);
                api->device_synchronize();
                auto t0 = clk::now();
                {
                    model::PagedForwardContext ctx(ids, 0, table, pool);
                    auto logits = model::transformer_forward(fcfg, ctx, exec, nullptr);
                    (void)argmax.sample(logits);              // reads the token back: waits for the step
                }
                const double t = ms_since(t0);
                if (r >= warm) ms.push_back(t);
                alloc.free_sequence(table);
            }
            std::sort(ms.begin(), ms.end());
            std::printf("prefill %d %.4f %.4f %.4f\n", n, ms[ms.size() / 2], ms.front(), ms.back());
        } else if (f[0] == "decode") {
            const int B = std::atoi(f[1].c_str()), ctx0 = std::atoi(f[2].c_str()), steps = std::atoi(f[3].c_str()),
                      warm = std::atoi(f[4].c_str());
            std::vector<std::unique_ptr<InferenceRequest>> reqs;
            for (int b = 0; b < B; ++b) {
                auto req = std::make_unique<InferenceRequest>();
                req->request_id = (uint64_t)b;
                req->input_ids = random_ids(ctx0, (int)V);
                req->own_block_table(alloc.allocate_sequence(ctx0 + steps + warm + 1));
                // the prompt, in portions of 512 as the reference's scheduler cuts it
                for (int start = 0; start < ctx0; start += 512) {
                    const int n = std::min(512, ctx0 - start);
                    std::vector<int> part(req->input_ids.begin() + start, req->input_ids.begin() + start + n);
                    alloc.ensure_blocks(req->block_table(), start + n);
                    model::PagedForwardContext ctx(part, start, req->block_table(), pool);
                    auto logits = model::transformer_forward(fcfg, ctx, exec, nullptr);
                    if (start + n == ctx0) req->last_token = argmax.sample(logits);
                    req->block_table().seq_len = start + n;
                }
                reqs.push_back(std::move(req));
            }
            api->device_synchronize();
            clk::time_point t0;
            for (int s = 0; s < warm + steps; ++s) {
                if (s == warm) { api->device_synchronize(); t0 = clk::now(); }
                ScheduledBatch batch;
                for (auto& r : reqs) {
                    alloc.ensure_blocks(r->block_table(), r->block_table().seq_len + 1);
                    batch.decode_requests.push_back(r.get());
                }
                auto bctx = batch.build_context();
                model::PagedForwardContext ctx(bctx, alloc);
                auto* sc = (B == 1) ? scratch.get() : nullptr;       // the serving loop's rule for the scratch buffers
                auto logits = model::transformer_forward(fcfg, ctx, exec, sc);
                int offset = 0;
                for (auto& r : reqs) {
                    auto row = logits->slice(0, offset, offset + 1);
                    const int tok = argmax.sample(row);
                    r->output_ids.push_back(tok);
                    r->last_token = tok;
                    r->generated_count++;
                    r->block_table().seq_len++;
                    ++offset;
                }
            }
            api->device_synchronize();
            const double total = ms_since(t0);
            std::printf("decode %d %d %d %.5f %.3f\n", B, ctx0, steps, total / steps, total);
            for (auto& r : reqs) alloc.free_sequence(r->block_table());
        }
        std::fflush(stdout);
    }
    return 0;
}
