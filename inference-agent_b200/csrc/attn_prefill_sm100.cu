#include "ingot_internal.cuh"
int launch_attn_prefill_sm100(ingot_kv*, int, const void*, int, void*, int, int, int, int, cudaStream_t) {
    ingot_set_error("tcgen05 prefill not built yet");
    return INGOT_ERR_UNSUPPORTED;
}
void free_prefill_sm100_state(ingot_kv*) {}
