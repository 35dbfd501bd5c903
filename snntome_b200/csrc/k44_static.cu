// k44b_wave_forward_static: one tensor-core wave with no device-memory allocation anywhere in the call.
//
// Who needs this: processes in which the library is not allowed to allocate device memory on its own —
// a serving process whose every byte of HBM belongs to an arena owned by the host framework, a caller
// running under a fixed memory budget that must not move at run time, or a latency-critical loop that
// cannot afford the implicit device-wide synchronisation of cudaMalloc / cudaFree. Such a caller hands in
// device pointers it owns (canvas, packed weights, run table, bias); the only extra memory the split-K wave
// kernel needs — FP32 partial-sum tiles, per-tile arrival counters and a status word — lives in the
// fixed-size array below, which is part of the library image on every GPU that loads it.
//
// In host code the array's name is only a stand-in: its device address is fetched once per device with
// cudaGetSymbolAddress (that device being current) and that pointer is what the kernel receives.
#include <cstdio>
#include <mutex>

#include "../../include/k44b.h"
#include "k44_exec.hpp"

namespace {

constexpr uint32_t kMaxTiles = K44B_STATIC_MAX_TILES;                 // 128-neuron x 64-column output tiles per call
constexpr size_t kStatusBytes = 256;                                   // status word (+ padding)
constexpr size_t kCounterBytes = ((size_t)kMaxTiles * 4 + 255) / 256 * 256;
constexpr size_t kTileBytes = 64u * k44b::kTileM * sizeof(float);      // 32 KiB of FP32 partial sums per tile
constexpr size_t kStaticBytes = kStatusBytes + kCounterBytes + (size_t)kMaxTiles * kTileBytes;

// [status | counters | partial-sum tiles]; about 2 MiB, held by every GPU that loads the library until exit.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;       // driver entry point, looked up once (first set-up)

struct DeviceSlot {
    bool ready = false;
    unsigned char *base = nullptr;   // device address of g_static_scratch on this device
    int num_sms = 0;
};

constexpr int kMaxDevices = 64;
DeviceSlot g_slots[kMaxDevices];
std::mutex g_mutex;
thread_local std::string g_static_error;

int fail(const std::string &m) {
    g_static_error = m;
    return -1;
}

// Once per device, with that device current: resolve the array's device address, opt the kernels in to
// large dynamic shared memory and clear the array. Nothing here allocates.
int setup_current_device(DeviceSlot **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail("device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceSlot &s = g_slots[dev];
    if (!s.ready) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return fail(std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        if (major != 10) return fail("current device is not sm_100: kernels are built for B200 only");
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) return fail(std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        e = cudaDeviceGetAttribute(&s.num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        if (!g_encode) {
            void *fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn)
                return fail("cuTensorMapEncodeTiled is not available from the driver");
            g_encode = (EncodeTiledFn)fn;
        }
        e = k44b::umma_kernel_setup();
        if (e != cudaSuccess) return fail(std::string("kernel attribute setup: ") + cudaGetErrorString(e));
        e = cudaMemset(ptr, 0, kStaticBytes);
        if (e != cudaSuccess) return fail(std::string("clearing the static scratch: ") + cudaGetErrorString(e));
        s.base = static_cast<unsigned char *>(ptr);
        s.ready = true;
    }
    *out = &s;
    return 0;
}

int encode_canvas_map(CUtensorMap *map, void *canvas, uint64_t canvas_elems, uint32_t pitch, uint32_t box_h) {
    const cuuint64_t dims[2] = {pitch, canvas_elems / pitch};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch * 2u};
    const cuuint32_t box[2] = {64u, box_h};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, canvas, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : fail("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

}  // namespace

extern "C" {

int k44b_wave_forward_static(void *d_canvas, uint64_t canvas_elems, uint32_t pitch, const void *d_weights_tiled,
                             const uint32_t *d_box_rows, uint32_t rows_per_box, const uint16_t *d_bias, uint32_t cout, uint32_t group,
                             uint32_t fan_in, int act, uint64_t y_off, uint32_t k_splits, void *stream, char *err, uint32_t err_capacity) {
    using namespace k44b;
    auto report = [&](int rc) {
        if (rc != 0 && err && err_capacity) {
            std::snprintf(err, err_capacity, "%s", g_static_error.c_str());
        }
        return rc;
    };
    if (!d_canvas || !d_weights_tiled || !d_box_rows) return report(fail("null device pointer"));
    if (pitch == 0 || pitch % 64u) return report(fail("row pitch must be a multiple of 64"));
    if (cout == 0 || cout % 16u || fan_in == 0 || fan_in % 8u) return report(fail("cout must be a multiple of 16 and fan-in a multiple of 8"));
    if (rows_per_box != 8 && rows_per_box != 16 && rows_per_box != 32 && rows_per_box != 64) return report(fail("rows per box must be 8, 16, 32 or 64"));
    if (group == 0 || cout % group || !(group % kTileM == 0u || group == cout)) return report(fail("group must be a multiple of 128 neurons or the whole wave"));
    if (y_off % 8u || y_off + (uint64_t)cout * pitch > canvas_elems) return report(fail("output rows leave the canvas or are misaligned"));
    if (act < 0 || act > ACT_GELU) return report(fail("unknown activation"));
    const uint32_t mtiles = (cout + kTileM - 1) / kTileM, tiles64 = pitch / 64u, tiles = mtiles * tiles64;
    const uint32_t kstages = (fan_in + kStageK - 1) / kStageK;
    if (tiles > kMaxTiles)
        return report(fail("wave needs " + std::to_string(tiles) + " output tiles of 128 neurons x 64 columns; the static scratch holds at most " +
                           std::to_string(kMaxTiles) + " (K44B_STATIC_MAX_TILES)"));
    if (k_splits == 0 || k_splits > kstages) return report(fail("k_splits must be between 1 and ceil(fan_in / 64)"));

    cudaStream_t s = (cudaStream_t)stream;
    {   // every call reads the status word back and waits for the stream: none of that may be recorded into a graph
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)
            return report(fail("the stream is being captured: this call synchronises the stream and cannot be part of a capture"));
    }
    DeviceSlot *slot = nullptr;
    if (setup_current_device(&slot) != 0) return report(-1);
    uint32_t *status = reinterpret_cast<uint32_t *>(slot->base);
    uint32_t *counters = reinterpret_cast<uint32_t *>(slot->base + kStatusBytes);
    float *partial = reinterpret_cast<float *>(slot->base + kStatusBytes + kCounterBytes);

    // The array is shared by every call and keeps what the last one left: start from zero for the part used.
    cudaError_t e = cudaMemsetAsync(slot->base, 0, kStatusBytes + kCounterBytes, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(partial, 0, (size_t)tiles * kTileBytes, s);
    if (e != cudaSuccess) return report(fail(std::string("clearing the static scratch: ") + cudaGetErrorString(e)));

    WaveArgs a;
    a.w_tiles = static_cast<const uint4 *>(d_weights_tiled);
    a.gather = d_box_rows;
    a.bias = reinterpret_cast<const __half *>(d_bias);
    a.canvas = static_cast<__half *>(d_canvas);
    a.status = status;
    a.canvas_elems = canvas_elems;
    a.y_off = y_off;
    a.cout = cout; a.group = group; a.fan_in = fan_in;
    a.mtiles_per_group = group == cout ? mtiles : group / kTileM;
    a.num_kstages = kstages;
    a.pitch = pitch; a.num_col_tiles64 = tiles64;
    a.gather_mode = GATHER_BOX;
    a.box_h = rows_per_box; a.boxes_per_group = kstages * (kStageK / rows_per_box);
    a.act = act; a.has_residual = 0;
    a.kstages_per_split = (kstages + k_splits - 1) / k_splits;
    a.k_splits = (kstages + a.kstages_per_split - 1) / a.kstages_per_split;
    a.scratch = partial;
    a.counters = counters;
    UmmaDesc d = make_umma_desc(64);
    d.small_wave = 1;
    CUtensorMap map;
    if (encode_canvas_map(&map, d_canvas, canvas_elems, pitch, rows_per_box) != 0) return report(-1);
    e = launch_wave_umma(a, d, map, slot->num_sms, s);
    if (e != cudaSuccess) return report(fail(std::string("kernel launch: ") + cudaGetErrorString(e)));
    uint32_t st = 0;
    e = cudaMemcpyAsync(&st, status, sizeof st, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return report(fail(std::string("wave execution: ") + cudaGetErrorString(e)));
    if (st != 0) return report(fail(std::string("kernel status: ") + status_string(st)));
    return 0;
}

}  // extern "C"
