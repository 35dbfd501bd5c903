// Streaming tcgen05 wave kernel, tiles of 128 columns: instantiations and launch dispatch (see k44_stream_kernel.cuh).
#include "k44_stream_kernel.cuh"

namespace k44b {

cudaError_t launch_wave_umma_n128(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s) {
    if (a.box_h == 1u)                   // scattered single rows
        return d.rows_mode == 2u ? umma_launch<128, 0, 2>(a, d, tmap, num_sms, s) : umma_launch<128, 0, 1>(a, d, tmap, num_sms, s);
    return umma_launch<128, 0>(a, d, tmap, num_sms, s);
}

cudaError_t umma_setup_n128() {
    cudaError_t e;
    if ((e = umma_attr<128, 0>()) != cudaSuccess) return e;
    if ((e = umma_attr<128, 0, 1>()) != cudaSuccess) return e;
    return umma_attr<128, 0, 2>();
}

}  // namespace k44b
