// Symbols that the reference's Qwen2 objects refer to but never call on this path (its mixture-of-experts layer).
#include "frontend/models/forward_config.hpp"
#include "zedinfer/activation.hpp"
#include <stdexcept>
namespace zedinfer::model {
struct DecodeScratch;
void moe_layer_forward(const ModelForwardConfig&, tensor_t, tensor_t, int, const ExecutorConfig&, DecodeScratch*) {
    throw std::runtime_error("moe_layer_forward is not part of this build");
}
}  // namespace zedinfer::model
