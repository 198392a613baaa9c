// Compile-and-link probe for include/cuqwen_compat.hpp: a program shaped like the reference's own main loop
// (load_weights -> malloc_qwen_state -> qwen_forward -> free_*) and a few launch_* calls must build unchanged.
// With no argument it only checks static facts and exits; given a model file it would run on a GPU.
#include "cuqwen_compat.hpp"

static_assert(QwenConfig::magic == 0x5157454E, "magic");
static_assert(QwenConfig::dim % QUANT_GROUP_SIZE == 0, "dim");

int main(int argc, char** argv) {
    printf("%s %s %s dim=%d layers=%d quant=%d stride=%d\n", QwenConfig::model_name, MODEL_TAG, QwenConfig::bin_path, QwenConfig::dim, QwenConfig::n_layers,
           QwenConfig::quant_type, (int)WEIGHT_ROW_STRIDE(QwenConfig::dim));
    if (argc < 2) return 0;
    QwenWeights weights;
    QwenConfig config = load_weights(argv[1], weights);
    QwenState state;
    malloc_qwen_state(config, state);
    int tok = 1;
    for (int pos = 0; pos < 4; ++pos) tok = qwen_forward(tok, pos, config, state, weights);
    const int more[3] = {5, 6, 7};
    qwen_prefill(more, 3, 4, config, state, weights);              // the shim's batched prefill: cache rows 4..6
    tok = qwen_forward(tok, 7, config, state, weights);
    launch_rmsnorm(state.x, weights.norm_weight, state.att, config.dim, __float2half(config.norm_eps));
    launch_gemv_add_fp16(weights.layers[0].o_proj_weight, weights.layers[0].o_proj_scale, state.xb, state.x, config.dim, config.n_heads * config.head_dim);
    launch_argmax(state.logits, state.d_sampled_token, config.vocab_size);
    // what harnesses of the reference poke directly must be valid device memory here as well
    int dev_tok = -1, dev_pos = -1;
    CUDA_CHECK(cudaStreamSynchronize(0));
    CUDA_CHECK(cudaMemcpy(&dev_tok, state.d_sampled_token, sizeof(int), cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(&dev_pos, state.d_pos, sizeof(int), cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemset(state.up, 0, (size_t)config.intermediate_size * sizeof(half)));
    CUDA_CHECK(cudaMemset(state.mlp_out, 0, (size_t)config.dim * sizeof(half)));
    CUDA_CHECK(cudaMemset(state.d_partial_out, 0, 16));
    CUDA_CHECK(cudaMemset(state.d_partial_max, 0, 16));
    CUDA_CHECK(cudaMemset(state.d_token, 0, sizeof(int)));
    CUDA_CHECK(cudaMemset(state.d_history_len, 0, sizeof(int)));
    if (!state.stream || dev_pos != 7 || dev_tok < 0 || dev_tok >= config.vocab_size) { printf("state fields: pos %d token %d\n", dev_pos, dev_tok); return 1; }
    static_assert(ATTN_KEYS_CAP > 0 && GEMV_WARPS_PER_BLOCK == 8 && GEMV_WIDE_WARPS_PER_BLOCK >= 8 && ARGMAX_THREADS == 256, "knob names");
    printf("%d\n", tok);
    free_qwen_state(state);
    free_weights(weights, config);
    return 0;
}
