// Symbols the reference's CPU-only objects refer to but never call on this path (GPU scatter, MoE).
#include "frontend/models/forward_config.hpp"
#include "zedinfer/activation.hpp"
#include <stdexcept>
namespace zedinfer::model {
struct DecodeScratch;
void moe_layer_forward(const ModelForwardConfig&, tensor_t, tensor_t, int, const ExecutorConfig&, DecodeScratch*) {
    throw std::runtime_error("moe_layer_forward is not part of this build");
}
}  // namespace zedinfer::model
namespace zedinfer::ops::nvidia {
void scatter_paged_kv(const void*, const void*, void*, void*, const int*, int, int, int, unsigned long) {
    throw std::runtime_error("scatter_paged_kv (GPU) is not part of this build");
}
}  // namespace zedinfer::ops::nvidia
