// Drives the reference's own CPU forward (transformer_forward + PagedForwardContext + BlockPool) on a tiny
// Qwen2 model.  Input: a flat file of float32 tensors with a text index; output: float32 logits [T, V].
#include "backend/kvcache/block_pool.hpp"
#include "backend/tensor/tensor.hpp"
#include "frontend/models/forward_config.hpp"
#include "frontend/models/paged_forward_context.hpp"
#include "frontend/models/qwen2.hpp"
#include "zedinfer/activation.hpp"

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <sstream>
#include <vector>

namespace zedinfer::model {
tensor_t transformer_forward(const ModelForwardConfig& model, PagedForwardContext& ctx, const ExecutorConfig& exec_config,
                             DecodeScratch* scratch, tensor_t input_embeds);
}
using namespace zedinfer;

int main(int argc, char** argv) {
    if (argc < 5) { std::cerr << "usage: ref_forward index.txt weights.bin out.bin block_size [chunk]\n"; return 2; }
    std::ifstream idx(argv[1]);
    std::ifstream bin(argv[2], std::ios::binary);
    const int block_size = std::atoi(argv[4]);
    const int chunk = argc > 5 ? std::atoi(argv[5]) : 0;
    model::ModelConfig base;
    std::vector<int> ids;
    auto weights = std::make_unique<model::ModelWeights>();
    std::string line;
    while (std::getline(idx, line)) {
        std::istringstream ss(line);
        std::string kind;
        ss >> kind;
        if (kind == "config") {
            size_t tie;
            ss >> base.hidden_size >> base.intermediate_size >> base.vocab_size >> base.num_hidden_layers
               >> base.num_attention_heads >> base.num_key_value_heads >> base.head_dim >> base.rms_norm_eps
               >> base.rope_theta >> tie;
            base.tie_word_embeddings = tie != 0;
            base.max_position_embeddings = 4096;
            base.model_type = "qwen2";
            base.torch_dtype = "float32";
        } else if (kind == "ids") {
            int v;
            while (ss >> v) ids.push_back(v);
        } else if (kind == "tensor") {
            std::string name;
            size_t nd;
            ss >> name >> nd;
            std::vector<size_t> shape(nd);
            size_t numel = 1;
            for (auto& s : shape) { ss >> s; numel *= s; }
            std::vector<float> buf(numel);
            bin.read(reinterpret_cast<char*>(buf.data()), numel * sizeof(float));
            auto t = Tensor::create(shape, ZEDINFER_DTYPE_F32, ZEDINFER_DEVICE_CPU, 0);
            t->load(buf.data());
            weights->add_tensor(name, t);
        }
    }
    if (base.tie_word_embeddings && !weights->has_tensor("lm_head.weight"))
        weights->add_tensor("lm_head.weight", weights->get_tensor("embed_tokens.weight"));
    model::Qwen2Config qcfg(base);
    qcfg.sliding_window = 4096; qcfg.max_window_layers = 21; qcfg.use_sliding_window = false;
    model::Qwen2Model qwen(qcfg, std::move(weights));
    auto fcfg = qwen.forward_config();

    kvcache::BlockConfig bc;
    bc.block_size = block_size; bc.num_kv_heads = (int)base.num_key_value_heads; bc.head_dim = (int)base.head_dim;
    bc.dtype = ZEDINFER_DTYPE_F32;
    const int T = (int)ids.size();
    const int blocks = ((T + block_size - 1) / block_size + 1) * (int)base.num_hidden_layers;
    kvcache::BlockPool pool(bc, blocks, ZEDINFER_DEVICE_CPU, 0);
    kvcache::BlockAllocator alloc(pool, (int)base.num_hidden_layers);
    auto table = alloc.allocate_sequence(T);
    ExecutorConfig exec(ZEDINFER_DEVICE_CPU, 0, ZEDINFER_DTYPE_F32, 4096);

    std::ofstream out(argv[3], std::ios::binary);
    const int step = chunk > 0 ? chunk : T;
    for (int start = 0; start < T; start += step) {
        const int n = std::min(step, T - start);
        std::vector<int> part(ids.begin() + start, ids.begin() + start + n);
        model::PagedForwardContext ctx(part, start, table, pool);
        auto logits = model::transformer_forward(fcfg, ctx, exec, nullptr, nullptr);
        table.seq_len = start + n;
        out.write(reinterpret_cast<const char*>(logits->data()), (size_t)n * base.vocab_size * sizeof(float));
    }
    std::cerr << "ref_forward: " << T << " tokens, vocab " << base.vocab_size << "\n";
    return 0;
}
