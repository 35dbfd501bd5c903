/* libk44wavec.so — drop-in C ABI of the SNNtome wave compiler/executor library.
 *
 * Same names, argument meaning and 0 / -1 result convention as the reference's `extern "C"` block
 * (wavec/k44_wave_executor.cu:642-988) so that the reference's ctypes binding (wavec/wavec.py:28-132)
 * loads this library unchanged. Differences, all on the safe side:
 *   - a GPU runtime error never terminates the process (the reference calls exit(), :54-62): the
 *     call returns -1 and k44b_last_error() (k44b.h) holds the reason;
 *   - 1-D token graphs compile: Input / linear (1x1 convolution) / split / slice / concat / RMSNorm / SwiGLU /
 *     rotary + grouped-query attention. 2-D image graphs (one input with h > 1, w a multiple of 4) compile: convolutions
 *     1x1 (stride 1, pad 0) and 3x3 (pad 1, stride 1 or 2) with bias / activation / residual, split / slice / concat,
 *     max-pool 2x2 stride 2 and 5x5 stride 1 pad 2, nearest 2x upsampling, 2x2 stride-2 transposed convolution. Planes are
 *     stored with one halo row above and below and four halo elements left (kernels/common/kernel44_valu_pack.cuh:30-103);
 *     wavec_gpu_infer_f32 takes and returns dense [c][h][w] FP32 images ([frame][c][h][w] after wavec_set_batch_size(frames)).
 *     A call outside that set (flatten, other kernel sizes, mixing the two kinds of graph) returns -1 and leaves the graph unchanged;
 *   - activation value 5 selects GELU in addition to the reference's 0-4. The tensor-core kernels evaluate it
 *     as v / (1 + exp(-v P(v^2))) with a fitted quadratic P, at most 2.6e-5 (absolute) away from the erf form;
 *     the FP32-FMA and mma.sync kernels call erff. Both lie inside the output tolerance (rtol 2e-3, atol 1e-3)
 *     for every FP16 pre-activation (checked by a sweep over all of them).
 * Not thread-safe per handle, like the reference.
 */
#ifndef K44WAVEC_H
#define K44WAVEC_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference: wavec/k44_wave_executor.cu:644 */
void *wavec_create(int max_B_per_wave, int default_S, int kv_cache_max_seq, int fold_rmsnorm_gamma);
/* :655 — also frees the GPU state */
void wavec_destroy(void *handle);
/* :669 — frees the GPU state only */
int wavec_gpu_release(void *handle);

/* :685 — is_1d (h == 1) token inputs, or one image input with h > 1 and w a multiple of 4 */
int wavec_add_input(void *handle, const char *name, int c, int h, int w, int is_1d);
/* :694 — not built (no consumer on the wave path): returns -1 */
int wavec_add_flatten(void *handle, const char *name, const char *in_tensor, const char *out_tensor);
/* :704 — token graphs: kh == kw == 1, stride 1, pad 0 (a linear). Image graphs: 1x1 / stride 1 / pad 0 and 3x3 / pad 1 /
 * stride 1 or 2; weights [cout][cin][kh][kw]. Otherwise -1 */
int wavec_add_conv2d(void *handle, const char *name, const char *in_tensor, const char *out_tensor, int cin, int cout,
                     int kh, int kw, int stride, int pad, int act, const float *w_f32, const float *bias_f32,
                     const char *residual_tensor);
/* :718 */
int wavec_add_conv2d_f16(void *handle, const char *name, const char *in_tensor, const char *out_tensor, int cin, int cout,
                         int kh, int kw, int stride, int pad, int act, const uint16_t *w_f16, const float *bias_f32,
                         const char *residual_tensor);
/* :733 — weights [dout][din] FP32, converted to FP16 round-to-nearest-even; arrays are copied */
int wavec_add_linear_f32(void *handle, const char *name, const char *in_tensor, const char *out_tensor, int din, int dout,
                         int act, const float *w_f32, const float *bias_f32, const char *residual_tensor);
/* :740 */
int wavec_add_linear_f16(void *handle, const char *name, const char *in_tensor, const char *out_tensor, int din, int dout,
                         int act, const uint16_t *w_f16, const float *bias_f32, const char *residual_tensor);
/* :747 — bf16 -> f32 -> f16 */
int wavec_add_linear_bf16(void *handle, const char *name, const char *in_tensor, const char *out_tensor, int din, int dout,
                          int act, const uint16_t *w_bf16, const float *bias_f32, const char *residual_tensor);
/* :761, :773, :783 — image graphs only. upconv2x2: weights [cout][cin][4] with the output phase 2 * (y & 1) + (x & 1)
 * innermost; maxpool: (k, stride, pad) = (2, 2, 0) or (5, 1, 2) */
int wavec_add_upconv2x2(void *handle, const char *name, const char *in_tensor, const char *out_tensor, int cin, int cout,
                        const float *w_f32, const float *bias_f32);
int wavec_add_maxpool(void *handle, const char *name, const char *in_tensor, const char *out_tensor, int k, int stride, int pad);
int wavec_add_upsample2x(void *handle, const char *name, const char *in_tensor, const char *out_tensor);
/* :793, :803, :813 — element-wise / attention commands between the waves (kernels/common/kernel44_valu_pack.cuh:104-248);
 * an RMSNorm scale is folded into the linears that consume it when fold_rmsnorm_gamma was set at wavec_create */
int wavec_add_rmsnorm(void *handle, const char *name, const char *in_tensor, const char *out_tensor, int dim, float eps,
                      const float *gamma_f32, int pre_folded);
int wavec_add_swiglu(void *handle, const char *name, const char *gate_tensor, const char *up_tensor, const char *out_tensor);
int wavec_add_rope_gqa_attn(void *handle, const char *name, const char *q_tensor, const char *k_tensor, const char *v_tensor,
                            const char *out_tensor, int h_q, int h_kv, int head_dim, float rope_theta, int llama3_scaling);
/* :826, :841, :860 — zero-copy channel views */
int wavec_add_split(void *handle, const char *name, const char *in_tensor, int num_outs, const char **out_tensors);
int wavec_add_slice(void *handle, const char *name, const char *in_tensor, int num_outs, const char **out_tensors,
                    const int *slice_sizes);
int wavec_add_concat(void *handle, const char *name, int num_ins, const char **in_tensors, const char *out_tensor);

/* :875, :884, :894, :904 — the setters mark the plan as not compiled */
int wavec_set_output(void *handle, const char *out_tensor);
int wavec_set_reuse_canvas(void *handle, int reuse_canvas);
int wavec_set_batch_size(void *handle, int batch_size);
int wavec_set_target_preset(void *handle, const char *preset_name);

/* :914 */
int wavec_compile(void *handle);
/* :923 — pointer into a string owned by the handle, valid until the next compile; compiles lazily */
const char *wavec_get_summary_json(void *handle);
/* :931 — include_canvas is ignored (canvas pages are never written), as in the reference */
int wavec_save_tcff_ex(void *handle, const char *tcff_path, const char *model_prefix, int include_canvas, int include_geometry);
/* :944 */
int wavec_save_tcff(void *handle, const char *tcff_path, const char *model_prefix);
/* :948 — fills the compiled plan's weights / bias (and gather table when the canvas size matches) */
int wavec_load_tcff_weights(void *handle, const char *tcff_path);
/* :956 — packs the plan onto the current CUDA device (device 0 unless k44b_set_device was called) */
int wavec_gpu_init_plan(void *handle);
/* :972 — h_in dense FP32 [C][1][W]; h_out dense FP32; out_gpu_ms = device time of the waves only */
int wavec_gpu_infer_f32(void *handle, const float *h_in, int in_elems, float *h_out, int out_elems, float *out_gpu_ms);

#ifdef __cplusplus
}
#endif
#endif
