// Cross-GPU signalling latency probe for neuron-sharded plans: two ranks bounce a counter word between their sync blocks
// over NVLink, optionally with a payload stored into the peer's canvas before every signal — the same sequence a sharded
// wave launch ends with (rows to the peer, one system-scope fence, one count word) and the next one starts with (poll the
// own word). The measured round trip is what every dependent launch of a sharded step has to pay at least once, so it is
// the floor a step's time is compared with. Every wait is bounded; nothing here allocates or frees.
#include "k44_kernels.cuh"

namespace k44b {

__global__ void __launch_bounds__(128) k44_peer_pingpong_kernel(uint32_t *own_word, uint32_t *peer_word, uint4 *peer_payload, uint32_t payload_vecs,
                                                                uint32_t initiator, uint32_t iters, uint32_t base, unsigned long long limit,
                                                                unsigned long long *out) {
    __shared__ uint32_t ok_s;
    const uint32_t tid = threadIdx.x;
    if (tid == 0) ok_s = 1u;
    __syncthreads();
    auto wait_for = [&](uint32_t want) -> bool {
        const long long t0 = clock64();
        for (;;) {
            uint32_t v;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(own_word) : "memory");
            if ((int32_t)(v - want) >= 0) break;
            if ((unsigned long long)(clock64() - t0) > limit) return false;
        }
        __threadfence_system();
        return true;
    };
    auto send = [&](uint32_t value) {           // all threads: payload, then one fence and the word from thread 0
        for (uint32_t v = tid; v < payload_vecs; v += blockDim.x) peer_payload[v] = make_uint4(value, value, value, value);
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(peer_word), "r"(value) : "memory");
        }
    };
    unsigned long long t_begin = 0, t_end = 0;
    if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_begin));
    uint32_t done = 0;
    for (uint32_t i = 1; i <= iters; ++i) {
        if (initiator) send(base + i);
        if (tid == 0 && !wait_for(base + i)) ok_s = 0u;
        __syncthreads();
        if (!ok_s) break;
        if (!initiator) send(base + i);
        ++done;
    }
    if (tid == 0) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_end));
        out[0] = t_end - t_begin;
        out[1] = done;
    }
}

cudaError_t launch_peer_pingpong(uint32_t *own_word, uint32_t *peer_word, void *peer_payload, uint32_t payload_bytes, bool initiator, uint32_t iters,
                                 uint32_t base, unsigned long long wait_cycles, unsigned long long *d_out, cudaStream_t s) {
    k44_peer_pingpong_kernel<<<1, 128, 0, s>>>(own_word, peer_word, (uint4 *)peer_payload, payload_bytes / 16u, initiator ? 1u : 0u, iters, base, wait_cycles, d_out);
    return cudaGetLastError();
}

}  // namespace k44b
