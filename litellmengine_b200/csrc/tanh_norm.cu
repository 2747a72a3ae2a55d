// The norm that computes no mean and no variance ("dynamic tanh"):  n(v)[i] = tanh(alpha * v[i]) * w[i] + b[i],
// alpha one learned number, w and b vectors, everything in 32-bit.  Being elementwise it joins the residual add
// on both sides, so a layer that norms a sublayer's output AND the next sublayer's input needs one kernel between
// two sublayers:
//
//     v      = h[row] + post(y[row])            post = the norm on the sublayer's output (none: y joins as it is)
//     h[row] = v                                (with write_h; the stream is float32)
//     out    = pre(v)                           pre = the norm in front of the next sublayer, stored in the compute dtype
//
// y may be absent (then v = h[row]), float32 or bfloat16, and may come as the `parts` k-splits of a product,
// `part_stride` elements apart, added in order as they are read.  `rows` (optional) picks which rows are read, so
// a model's final norm runs only where logits are wanted (h is then left alone).  The three alphas are read from
// device memory: they are tensors of the model.
#include "common.cuh"

#define TN_THREADS 128

template <typename TY, typename TO>
__global__ void tanh_norm_kernel(float* __restrict__ h, const TY* __restrict__ y, long long y_stride, int parts,
                                 long long part_stride, const float* __restrict__ post_alpha,
                                 const float* __restrict__ post_w, const float* __restrict__ post_b,
                                 const float* __restrict__ pre_alpha, const float* __restrict__ pre_w,
                                 const float* __restrict__ pre_b, TO* __restrict__ out,
                                 const int32_t* __restrict__ rows, int hidden, int vec, int write_h) {
    // the norms' numbers are the model's: read before the wait for the kernel that produces h and y
    const float a_post = post_alpha ? post_alpha[0] : 1.0f;
    const float a_pre = pre_alpha ? pre_alpha[0] : 1.0f;
    pdl_begin();
    const size_t src = rows ? static_cast<size_t>(rows[blockIdx.x]) : blockIdx.x;
    float* hr = h + src * hidden;
    const TY* yr = y ? y + src * y_stride : nullptr;
    TO* orow = out ? out + static_cast<size_t>(blockIdx.x) * hidden : nullptr;
    if (vec) {
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < hidden; i += gridDim.y * blockDim.x * 8) {
            float v[8];
            load8(hr + i, v);
            if (yr) {
                float s[8];
                load8(yr + i, s);
                for (int part = 1; part < parts; ++part) {
                    float more[8];
                    load8(yr + part * part_stride + i, more);
#pragma unroll
                    for (int u = 0; u < 8; ++u) s[u] += more[u];
                }
                if (post_w) {
                    float g[8], c[8];
                    load8(post_w + i, g);
                    load8(post_b + i, c);
#pragma unroll
                    for (int u = 0; u < 8; ++u) s[u] = tanhf(a_post * s[u]) * g[u] + c[u];
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] += s[u];
                if (write_h) store8(hr + i, v);
            }
            if (orow) {
                float g[8], c[8];
                load8(pre_w + i, g);
                load8(pre_b + i, c);
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = tanhf(a_pre * v[u]) * g[u] + c[u];
                store8(orow + i, v);
            }
        }
        return;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) {
        float v = hr[i];
        if (yr) {
            float s = to_f32(yr[i]);
            for (int part = 1; part < parts; ++part) s += to_f32(yr[part * part_stride + i]);
            if (post_w) s = tanhf(a_post * s) * post_w[i] + post_b[i];
            v += s;
            if (write_h) hr[i] = v;
        }
        if (orow) orow[i] = from_f32<TO>(tanhf(a_pre * v) * pre_w[i] + pre_b[i]);
    }
}

// h: float32 [*, hidden]; y: [*, hidden] with `y_stride` elements a row, or null; post_* / pre_*: float32 [1], [hidden],
// [hidden], or null (no norm on that side; without pre_w nothing is written to `out`); out: [num_rows, hidden].
extern "C" int llm_tanh_norm(float* h, const void* y, int y_dtype, long long y_stride, int parts, long long part_stride,
                             const float* post_alpha, const float* post_w, const float* post_b, const float* pre_alpha,
                             const float* pre_w, const float* pre_b, void* out, int out_dtype, const int32_t* rows,
                             int num_rows, int hidden, uintptr_t stream) {
    if (num_rows <= 0) return LLM_OK;
    if (hidden <= 0 || parts < 1 || (y && y_stride < hidden)) return LLM_REFUSED_SIZE;
    if ((post_w == nullptr) != (post_b == nullptr) || (post_w == nullptr) != (post_alpha == nullptr)) return LLM_REFUSED_SIZE;
    if ((pre_w == nullptr) != (pre_b == nullptr) || (pre_w == nullptr) != (pre_alpha == nullptr)) return LLM_REFUSED_SIZE;
    if ((out == nullptr) != (pre_w == nullptr)) return LLM_REFUSED_SIZE;
    if (!y) y_dtype = LLM_DT_F32;
    if (!out) out_dtype = LLM_DT_F32;
    const int write_h = y && !rows;
    const int vec = hidden % 8 == 0 && aligned16(h) && (!y || (aligned16(y) && y_stride % 8 == 0 && part_stride % 8 == 0)) &&
                    (!out || aligned16(out)) && (!post_w || (aligned16(post_w) && aligned16(post_b))) &&
                    (!pre_w || (aligned16(pre_w) && aligned16(pre_b)));
    const int per_block = TN_THREADS * (vec ? 8 : 1);
    int gy = (hidden + per_block - 1) / per_block;
    if (gy > 64) gy = 64;
    const dim3 grid(num_rows, gy);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define LAUNCH(TY, TO)                                                                                                  \
    launch_pdl((tanh_norm_kernel<TY, TO>), grid, dim3(TN_THREADS), 0, s, h, static_cast<const TY*>(y), y_stride, parts, \
               part_stride, post_alpha, post_w, post_b, pre_alpha, pre_w, pre_b, static_cast<TO*>(out), rows, hidden,   \
               vec, write_h)
    if (y_dtype == LLM_DT_F32 && out_dtype == LLM_DT_F32) LAUNCH(float, float);
    else if (y_dtype == LLM_DT_F32 && out_dtype == LLM_DT_BF16) LAUNCH(float, bf16);
    else if (y_dtype == LLM_DT_BF16 && out_dtype == LLM_DT_F32) LAUNCH(bf16, float);
    else if (y_dtype == LLM_DT_BF16 && out_dtype == LLM_DT_BF16) LAUNCH(bf16, bf16);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}
