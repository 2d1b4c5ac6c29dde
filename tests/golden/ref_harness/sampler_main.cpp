// Drives the reference's own GeneralSampler (src/frontend/sampler/sampler.cpp, CPU path) on rows of float32 logits:
// for each case it prints the truncated, renormalised distribution that sample() draws from (truncatedDist:
// repetition penalty, temperature, softmax, top-k, top-p) as "token probability" pairs in the sampler's own order.
// Input (text): "vocab V", then cases "case temperature top_k top_p penalty n_recent r0 r1 ... " followed by a line
// of V logits.  Output (text): "case i n" then n lines "token prob".
#include "backend/tensor/tensor.hpp"
#include "frontend/sampler/sampler.hpp"

#include <cstdio>
#include <fstream>
#include <iostream>
#include <sstream>
#include <vector>

using namespace zedinfer;

int main(int argc, char** argv) {
    if (argc < 3) { std::cerr << "usage: ref_sampler cases.txt out.txt\n"; return 2; }
    std::ifstream in(argv[1]);
    std::ofstream out(argv[2]);
    out.precision(9);
    std::string word;
    size_t vocab = 0;
    in >> word >> vocab;
    int index = 0;
    while (in >> word) {
        float temperature, top_p, penalty;
        int top_k, n_recent;
        in >> temperature >> top_k >> top_p >> penalty >> n_recent;
        std::vector<int> recent(n_recent);
        for (auto& r : recent) in >> r;
        std::vector<float> logits(vocab);
        for (auto& v : logits) in >> v;
        sampler::SamplerParams params(temperature, top_k, top_p, 1u);
        params.repetition_penalty = penalty;
        sampler::GeneralSampler s(params);
        auto t = Tensor::create({vocab}, ZEDINFER_DTYPE_F32, ZEDINFER_DEVICE_CPU, 0);
        t->load(logits.data());
        auto dist = s.truncatedDist(t, &recent);
        out << "case " << index++ << " " << dist.size() << "\n";
        for (const auto& pr : dist) out << pr.second << " " << pr.first << "\n";
    }
    return 0;
}
