// The two kernels around a sublayer of a layer whose norm follows the sum and whose sublayers read the
// residual stream through a short causal convolution over time:
//
//   short_conv        u[t, c] = x[t, c] + sum_j w[c, j] * x_(t - taps + 1 + j)[c]       (j = 0 .. taps - 1)
//                     x is the float32 stream [T, W]; the rows of earlier tokens of the same request come from
//                     the step's own rows when the token's portion holds them, else from the request's kept
//                     rows, and are zero before the sequence's start; u is stored in the compute dtype (it
//                     feeds matrix products).  The arithmetic is 32-bit.
//   scaled_add_norm   x[t, :] <- rmsnorm(alpha * x[t, :] + y[t, :]) * w, in place, in 32-bit; y may be a product
//                     left as its k-splits (added in order while reading).  On the way the kernel keeps the
//                     OLD row x[t, :] (what the sublayer before this norm read through its convolution) for the
//                     request's next step, if the token is among the last taps - 1 of its portion.
//
// Kept rows.  Per request slot and sublayer a ring of R = taps - 1 rows of W floats; the row of the token at
// position p sits at ring row p mod R.  The convolution of a token at position p reads positions p - 1 .. p - R
// (R different ring rows); the ring is written by the norm kernel, which runs after the convolution of the same
// sublayer has read it, and only the last R tokens of a portion write (R different ring rows), so no row is
// written twice in a step and none is read after it was overwritten.  A portion may be cut anywhere and be as
// short as one token.
#include "common.cuh"

#define CN_THREADS 256

template <int V>
__device__ __forceinline__ void load_row(float (&v)[V], const float* p) {       // V == 4: one 16-byte load
    if constexpr (V == 4) {
        const float4 f = *reinterpret_cast<const float4*>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
        for (int u = 0; u < V; ++u) v[u] = p[u];
    }
}

// TT consecutive tokens a block (a step of many tokens: their index lookups and row loads are in flight together,
// which is what the kernel waits for; a short step takes TT = 1 and one block a token).  A row that does not exist
// (before the sequence's start) is not added; its load is pointed at the token's own row.
template <typename TO, int V, int TT>
__global__ void short_conv_kernel(
    const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out, const float* __restrict__ kept,
    long long kept_slot_stride, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start, int num_tokens, int width, int taps) {
    pdl_begin();
    const int t0 = blockIdx.x * TT;
    const int c = (blockIdx.y * CN_THREADS + threadIdx.x) * V;
    if (c >= width) return;
    const int R = taps - 1;
    int tok[TT], q0[TT], pos[TT];
    const float* ring[TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        tok[i] = min(t0 + i, num_tokens - 1);               // a block's spare tokens repeat the last one and store nothing
        const int e = token_entry[tok[i]];
        q0[i] = entry_q_start[e];
        pos[i] = positions[tok[i]];
        ring[i] = kept ? kept + static_cast<size_t>(entry_slot[e]) * kept_slot_stride : nullptr;
    }
    float acc[TT][V], cur[TT][V];
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        load_row<V>(cur[i], x + static_cast<size_t>(tok[i]) * width + c);
#pragma unroll
        for (int u = 0; u < V; ++u) acc[i][u] = cur[i][u];
    }
    for (int back = R; back >= 1; --back) {                 // oldest first: the order of additions is fixed
        float wj[V], old[TT][V];
        bool there[TT];
#pragma unroll
        for (int u = 0; u < V; ++u) wj[u] = w[static_cast<size_t>(c + u) * taps + taps - 1 - back];
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            const float* src = x + static_cast<size_t>(tok[i]) * width + c;
            there[i] = true;
            if (tok[i] - back >= q0[i]) src = x + static_cast<size_t>(tok[i] - back) * width + c;
            else if (pos[i] - back >= 0 && ring[i]) src = ring[i] + static_cast<size_t>((pos[i] - back) % R) * width + c;
            else there[i] = false;                          // before the sequence's start: zero
            load_row<V>(old[i], src);
        }
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            if (there[i]) {
#pragma unroll
                for (int u = 0; u < V; ++u) acc[i][u] += wj[u] * old[i][u];
            }
        }
    }
    float wl[V];
#pragma unroll
    for (int u = 0; u < V; ++u) wl[u] = w[static_cast<size_t>(c + u) * taps + taps - 1];
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        if (t0 + i >= num_tokens) break;
#pragma unroll
        for (int u = 0; u < V; ++u) acc[i][u] += wl[u] * cur[i][u];
        TO* o = out + static_cast<size_t>(t0 + i) * width + c;
        if constexpr (V == 4 && sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(o) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        } else if constexpr (V == 4 && sizeof(TO) == 2) {
            __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc[i][0], acc[i][1]), hi2 = __floats2bfloat162_rn(acc[i][2], acc[i][3]);
            uint2 pk;
            pk.x = *reinterpret_cast<unsigned*>(&lo2);
            pk.y = *reinterpret_cast<unsigned*>(&hi2);
            *reinterpret_cast<uint2*>(o) = pk;
        } else {
#pragma unroll
            for (int u = 0; u < V; ++u) o[u] = from_f32<TO>(acc[i][u]);
        }
    }
}

extern "C" int llm_short_conv(const float* x, const float* w, void* out, int out_dtype, const float* kept,
                              long long kept_slot_stride, const int32_t* positions, const int32_t* token_entry,
                              const int32_t* entry_slot, const int32_t* entry_q_start, int num_tokens, int width,
                              int taps, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (width <= 0 || taps < 1 || (taps > 1 && !kept)) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bool four = width % 4 == 0 && aligned16(x) && aligned16(out) && (!kept || (aligned16(kept) && kept_slot_stride % 4 == 0));
    const int per = four ? 4 : 1;
    const bool many = four && num_tokens >= 256;            // four tokens a block
    const dim3 grid(many ? (num_tokens + 3) / 4 : num_tokens, (width + CN_THREADS * per - 1) / (CN_THREADS * per));
#define LAUNCH(TO, V, TT)                                                                                       \
    launch_pdl((short_conv_kernel<TO, V, TT>), grid, dim3(CN_THREADS), 0, s, x, w, static_cast<TO*>(out), kept,  \
               kept_slot_stride, positions, token_entry, entry_slot, entry_q_start, num_tokens, width, taps)
    if (out_dtype == LLM_DT_F32) { if (many) LAUNCH(float, 4, 4); else if (four) LAUNCH(float, 4, 1); else LAUNCH(float, 1, 1); }
    else if (out_dtype == LLM_DT_BF16) { if (many) LAUNCH(bf16, 4, 4); else if (four) LAUNCH(bf16, 4, 1); else LAUNCH(bf16, 1, 1); }
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}

// One block a token.  The row alpha * x + y is held in shared memory between the pass that sums its squares and the
// pass that scales it.
template <typename TY, bool VEC>
__global__ void scaled_add_norm_kernel(
    float* __restrict__ x, const TY* __restrict__ y, long long y_stride, int parts, long long part_stride,
    const float* __restrict__ w, float alpha, float eps, float* __restrict__ kept, long long kept_slot_stride, int ring_rows,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry, const int32_t* __restrict__ entry_slot,
    const int32_t* __restrict__ entry_q_start, const int32_t* __restrict__ entry_q_len, int width) {
    pdl_begin();
    extern __shared__ __align__(16) float row[];            // [width] + 33
    float* scratch = row + width;
    const int t = blockIdx.x;
    float* xr = x + static_cast<size_t>(t) * width;
    const TY* yr = y + static_cast<size_t>(t) * y_stride;
    float* keep = nullptr;
    if (kept && ring_rows > 0) {
        const int e = token_entry[t];
        if (t >= entry_q_start[e] + entry_q_len[e] - ring_rows)
            keep = kept + static_cast<size_t>(entry_slot[e]) * kept_slot_stride +
                   static_cast<size_t>(positions[t] % ring_rows) * width;
    }
    float ss = 0.0f;
    if (VEC) {                                              // four channels a thread, 16-byte loads; the same additions
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 old = *reinterpret_cast<const float4*>(xr + i);
            float add[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
            for (int z = 0; z < parts; ++z) {
                float v[4];
                if constexpr (sizeof(TY) == 4) {
                    const float4 f = *reinterpret_cast<const float4*>(yr + z * part_stride + i);
                    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                } else {
                    const uint2 u = *reinterpret_cast<const uint2*>(yr + z * part_stride + i);
                    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
                    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) add[u] += v[u];
            }
            const float4 v = make_float4(alpha * old.x + add[0], alpha * old.y + add[1], alpha * old.z + add[2], alpha * old.w + add[3]);
            if (keep) *reinterpret_cast<float4*>(keep + i) = old;
            *reinterpret_cast<float4*>(row + i) = v;
            ss += v.x * v.x;
            ss += v.y * v.y;
            ss += v.z * v.z;
            ss += v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float old = xr[i];
            float add = 0.0f;
            for (int z = 0; z < parts; ++z) add += to_f32(yr[z * part_stride + i]);
            const float v = alpha * old + add;
            if (keep) keep[i] = old;
            row[i] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / static_cast<float>(width) + eps);
    if (VEC) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + i), ww = *reinterpret_cast<const float4*>(w + i);
            *reinterpret_cast<float4*>(xr + i) = make_float4(v.x * inv * ww.x, v.y * inv * ww.y, v.z * inv * ww.z, v.w * inv * ww.w);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) xr[i] = row[i] * inv * w[i];
    }
}

extern "C" int llm_scaled_add_norm(float* x, const void* y, int y_dtype, long long y_stride, int parts,
                                   long long part_stride, const float* w, float alpha, float eps, float* kept,
                                   long long kept_slot_stride, int ring_rows, const int32_t* positions,
                                   const int32_t* token_entry, const int32_t* entry_slot, const int32_t* entry_q_start,
                                   const int32_t* entry_q_len, int num_tokens, int width, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (width <= 0 || parts < 1 || ring_rows < 0) return LLM_REFUSED_SIZE;
    const size_t smem = (static_cast<size_t>(width) + 33) * sizeof(float);
    if (smem > 200 * 1024) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int threads = width >= 2048 ? 512 : CN_THREADS;
    const bool vec = width % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(w) && y_stride % 4 == 0 && part_stride % 4 == 0 &&
                     (!kept || (aligned16(kept) && kept_slot_stride % 4 == 0));
#define LAUNCH(TY)                                                                                                 \
    do { if (vec) LAUNCH_V(TY, true); else LAUNCH_V(TY, false); } while (0)
#define LAUNCH_V(TY, VEC)                                                                                          \
    do {                                                                                                           \
        auto kern = scaled_add_norm_kernel<TY, VEC>;                                                                 \
        if (smem > 48 * 1024) {                                                                                    \
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                                                       static_cast<int>(smem));                                    \
            if (e != cudaSuccess) return static_cast<int>(e);                                                      \
        }                                                                                                          \
        launch_pdl(kern, dim3(num_tokens), dim3(threads), smem, s, x, static_cast<const TY*>(y), y_stride, parts,  \
                   part_stride, w, alpha, eps, kept, kept_slot_stride, ring_rows, positions, token_entry,          \
                   entry_slot, entry_q_start, entry_q_len, width);                                                 \
    } while (0)
    if (y_dtype == LLM_DT_F32) LAUNCH(float);
    else if (y_dtype == LLM_DT_BF16) LAUNCH(bf16);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
#undef LAUNCH_V
    return launch_status();
}
