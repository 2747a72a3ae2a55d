// Paged causal attention for any mix of tokens, any head size up to 256 in steps of 16, any
// head counts, float32 or bfloat16 — the kernel of the 32-bit path and the fallback of the
// bfloat16 path for sizes its tuned kernels do not take.
//
// For the query token t of the request in slot s at position p, head h (kv head h / group):
//     keys j in [lo, p],  lo = 0 or p - window + 1 with a window
//     s_j = (q . k_j) * scale;  softmax over j in 32-bit;  out = sum_j p_j v_j
// with the running-maximum form of src/ops/attention.cu:204-249 applied to tiles of 32 keys
// (the reference folds one key at a time; its paged kernel is src/ops/attention.cu:577-668).
// Keys and values are read straight from the pages through the device-resident block table,
// so prompt portions at any past length, single decoded tokens and mixed batches all take
// this one path; the step's own keys were written to the pages before this kernel runs.
//
// One thread block of AG_WARPS warps per (token, head).  The keys are cut into tiles of 32; warp w
// takes tiles w, w + AG_WARPS, ... : each lane scores one key of the tile (a 16-byte-vectorised dot
// product against q held in shared memory), the warp reduces max and sum, then every lane
// accumulates its output dimensions over the tile's values.  At the end the warps' running
// (maximum, sum, output) triples are merged through shared memory in warp order.  Which warp takes
// which tile depends only on (lo, p), never on the batch, so a position's result does not depend
// on how the work was cut.  (With one warp per (token, head) a decode step of 8 requests at a
// context of 4,096 kept two warps an SM busy: 5 ms a layer.)
//
// Keys and values may differ in width (dk, dv) and live in tensors of their own: `keys` [pages, nkv,
// page, dk] and `values` [pages, nkv, page, dv], each with its own page stride (the two halves of one
// [pages, 2, nkv, page, d] tensor are the special case dk == dv).  An optional output gate is applied
// before the store: out = o * sigmoid(gate[t, gate_off + h*dv + i]) * out_scale, and the output row
// may be a column range of a wider buffer (`out_stride`, `out_off`), which is how a layer that runs
// several mixers side by side collects their results for ONE output product.  With `gate_per_head` the
// gate holds one value per head (gate[t, gate_off + h]) instead of one per output channel.
//
// An optional learned bias by distance is added to the scaled score: s_j += dist_bias[min(p - j, len - 1),
// h], a float32 table [len, heads] indexed by the distance itself (whoever owns the table expands its
// bucketing into one row per distance up to the distance from which the row no longer changes).
// An analytic one instead (`log_r1`, `log_r2`, float32 [heads]): s_j -= r1[h] * ln(1 + r2[h] * (p - j)), which has
// no farthest row.  `head_scale` (float32 [heads]) multiplies a head's scaled scores (a learned temperature).
// `value_row_stride` (elements; 0: dv) lets the values be the first dv entries of rows that are wider, e.g. of
// the key rows themselves: a layer that caches one latent row per token, scores against all of it and sums its
// first part needs no second tensor.  Value widths above 256 take an instantiation with twice the accumulators.
// `keep_first` (with a window): the first so many keys of the sequence stay visible to every query behind them,
// at their true positions; the walk is then over the kept keys below the window and the window itself, as one
// list.  `has_sink`: one more term exp(sink_score) in the softmax's denominator that carries no value.
// With `rows` (int32 [num_tokens]) the kernel works on the listed tokens only (a step's single decoded tokens
// while its prompt portions take a tensor-core kernel); -1 entries pad the list.
#include "common.cuh"
#include <math_constants.h>

#define AG_WARPS 8
#define AG_MAX_D 256           // value width of the usual instantiation
#define AG_MAX_DV 512          // and of the wide one
#define AG_MAX_DK 1024         // key width (q is held in shared memory)

template <typename T, typename TC, int MAXDV>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q, T* __restrict__ out, const TC* __restrict__ keys, const TC* __restrict__ values,
    long long key_page_stride, long long value_page_stride,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    int num_tokens, int nq, int nkv, int d, int dv, int page_size, int window, float scale, int num_pages,
    const float* __restrict__ gate, long long gate_stride, int gate_off, float out_scale,
    long long out_stride, int out_off, int vec, int32_t* __restrict__ status,
    const float* __restrict__ dist_bias, int dist_len, int gate_per_head, const int32_t* __restrict__ rows,
    const float* __restrict__ head_scale, const float* __restrict__ log_r1, const float* __restrict__ log_r2,
    long long value_row_stride, int keep_first, int has_sink, float sink_score) {
    pdl_begin();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = blockIdx.x;
    const int listed = static_cast<int>(item / nq);
    const int h = static_cast<int>(item - static_cast<long long>(listed) * nq);
    const int t = rows ? rows[listed] : listed;          // `rows`: the tokens to work on (-1: padding of the list)
    if (t < 0) return;
    const int kvh = h / (nq / nkv);
    float* qs = smem;                                  // [d]
    float* merge = smem + d;                           // [AG_WARPS][dv + 2]: output, maximum, sum of each warp
    const T* qrow = q + (static_cast<size_t>(t) * nq + h) * d;
    const float hscale = head_scale ? scale * head_scale[h] : scale;
    for (int i = threadIdx.x; i < d; i += AG_WARPS * 32) qs[i] = to_f32(qrow[i]) * hscale;
    __syncthreads();
    const float r1 = log_r1 ? log_r1[h] : 0.0f, r2 = log_r1 ? log_r2[h] : 0.0f;

    const int pos = positions[t];
    const int slot = entry_slot[token_entry[t]];
    const int32_t* table = block_table + static_cast<size_t>(slot) * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const size_t khead = static_cast<size_t>(page_size) * d;        // one kv head inside a page of keys
    const size_t vrow = value_row_stride > 0 ? static_cast<size_t>(value_row_stride) : static_cast<size_t>(dv);
    const size_t vhead = static_cast<size_t>(page_size) * vrow;     // and inside a page of values

    float m = -CUDART_INF_F, l = 0.0f;
    float acc[MAXDV / 32];
#pragma unroll
    for (int r = 0; r < MAXDV / 32; ++r) acc[r] = 0.0f;

    // the keys a query walks: [0, head) kept from the sequence's start, then [lo, pos]
    const int head = keep_first < lo ? keep_first : lo;
    const int walk = head + pos - lo + 1;
    for (int base = 32 * warp; base < walk; base += 32 * AG_WARPS) {
        const int u0 = base + lane;
        const int j = u0 < head ? u0 : lo + (u0 - head);
        const bool valid = u0 < walk;
        long long voff = -1;
        float s = -CUDART_INF_F;
        if (valid) {
            const int logical = j / page_size;
            const int page = logical < table_stride ? table[logical] : -1;
            if (page < 0 || page >= num_pages) {
                if (atomicCAS(status, 0, 4) == 0) status[1] = t;
            } else {
                const TC* kr = keys + static_cast<long long>(page) * key_page_stride + kvh * khead +
                               static_cast<size_t>(j % page_size) * d;
                voff = static_cast<long long>(page) * value_page_stride + kvh * vhead +
                       static_cast<size_t>(j % page_size) * vrow;
                float dot = 0.0f;
                if (vec) {
                    for (int i = 0; i < d; i += 8) {
                        float kv[8];
                        load8(kr + i, kv);
#pragma unroll
                        for (int u = 0; u < 8; ++u) dot += qs[i + u] * kv[u];
                    }
                } else {
                    for (int i = 0; i < d; ++i) dot += qs[i] * to_f32(kr[i]);
                }
                s = dot;
                if (dist_bias) s += dist_bias[static_cast<size_t>(min(pos - j, dist_len - 1)) * nq + h];
                if (log_r1) s -= r1 * log1pf(r2 * static_cast<float>(pos - j));
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (voff >= 0) ? expf(s - m_new) : 0.0f;
        const float alpha = (m == -CUDART_INF_F) ? 0.0f : expf(m - m_new);
        l = l * alpha + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int r = 0; r < MAXDV / 32; ++r) acc[r] *= alpha;
        const int count = min(32, walk - base);
        const int regs = (dv + 31) >> 5;               // value entries a lane holds
        for (int jj = 0; jj < count; jj += 4) {       // four keys' value rows in flight: their loads do not wait for one another
            float pj[4];
            const TC* vr[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float pu = __shfl_sync(0xffffffffu, p, (jj + u) & 31);
                const long long vo = __shfl_sync(0xffffffffu, voff, (jj + u) & 31);
                const bool use = jj + u < count && vo >= 0;     // a key whose page was refused has no row
                pj[u] = use ? pu : 0.0f;
                vr[u] = values + (use ? vo : 0);
            }
#pragma unroll
            for (int r = 0; r < MAXDV / 32; ++r) {
                const int i = lane + 32 * r;
                if (r < regs && i < dv) {
                    float x[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) x[u] = to_f32(vr[u][i]);
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[r] += pj[u] * x[u];
                }
            }
        }
    }
    // merge the warps' partial results, in warp order (a warp without tiles has m = -inf, l = 0)
    float* mine = merge + warp * (dv + 2);
#pragma unroll
    for (int r = 0; r < MAXDV / 32; ++r) {
        const int i = lane + 32 * r;
        if (i < dv) mine[i] = acc[r];
    }
    if (lane == 0) { mine[dv] = m; mine[dv + 1] = l; }
    __syncthreads();
    float m_all = -CUDART_INF_F;
    for (int w2 = 0; w2 < AG_WARPS; ++w2) m_all = fmaxf(m_all, merge[w2 * (dv + 2) + dv]);
    float l_all = 0.0f;
    for (int w2 = 0; w2 < AG_WARPS; ++w2) {
        const float mw = merge[w2 * (dv + 2) + dv];
        if (mw != -CUDART_INF_F) l_all += merge[w2 * (dv + 2) + dv + 1] * expf(mw - m_all);
    }
    if (has_sink) l_all += expf(sink_score - m_all);   // the sink joins the sum; it has no value row (far above every
                                                       // score it overflows to infinity and the output to zero: its limit)
    T* orow = out + static_cast<size_t>(t) * out_stride + out_off + static_cast<size_t>(h) * dv;
    const float* grow = gate ? gate + static_cast<size_t>(t) * gate_stride + gate_off +
                                   (gate_per_head ? static_cast<size_t>(h) : static_cast<size_t>(h) * dv) : nullptr;
    const float inv = 1.0f / l_all;
    for (int i = threadIdx.x; i < dv; i += AG_WARPS * 32) {
        float o = 0.0f;
        for (int w2 = 0; w2 < AG_WARPS; ++w2) {
            const float mw = merge[w2 * (dv + 2) + dv];
            if (mw != -CUDART_INF_F) o += merge[w2 * (dv + 2) + i] * expf(mw - m_all);
        }
        o *= inv;
        if (grow) o *= 1.0f / (1.0f + expf(-grow[gate_per_head ? 0 : i]));
        orow[i] = from_f32<T>(o * out_scale);
    }
}

// The general entry point: keys and values by their own pointers, widths and page strides (in
// elements), optional output gate and scale, output as a column range of a wider buffer.
extern "C" int llm_paged_attention_generic_kv(
    const void* q, void* out, int dtype, const void* keys, const void* values, int cache_dtype,
    long long key_page_stride, long long value_page_stride, const int32_t* positions,
    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table, int table_stride,
    int num_tokens, int nq, int nkv, int d, int dv, int page_size, int window, float scale, int num_pages,
    const float* gate, long long gate_stride, int gate_off, float out_scale, long long out_stride, int out_off,
    int32_t* status, const float* dist_bias, int dist_len, int gate_per_head, const int32_t* rows,
    const float* head_scale, const float* log_r1, const float* log_r2, long long value_row_stride, int keep_first,
    int has_sink, float sink_score, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (keep_first < 0) return LLM_REFUSED_SIZE;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || d <= 0 || d > AG_MAX_DK || dv <= 0 || dv > AG_MAX_DV || page_size <= 0)
        return LLM_REFUSED_SIZE;
    if ((log_r1 == nullptr) != (log_r2 == nullptr) || value_row_stride < 0 || (value_row_stride > 0 && value_row_stride < dv))
        return LLM_REFUSED_SIZE;
    if (dist_bias && dist_len <= 0) return LLM_REFUSED_SIZE;
    const int esz = cache_dtype == LLM_DT_F32 ? 4 : 2;
    const int vec = (d % 8 == 0) && aligned16(keys) && (key_page_stride * esz) % 16 == 0;
    const size_t smem = (static_cast<size_t>(d) + static_cast<size_t>(AG_WARPS) * (dv + 2)) * sizeof(float);
    const long long items = static_cast<long long>(num_tokens) * nq;
    if (items > 0x7fffffffLL) return LLM_REFUSED_SIZE;
    const unsigned blocks = static_cast<unsigned>(items);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define LAUNCH(T, TC)                                                                              \
    if (dv > AG_MAX_D) LAUNCH_W(T, TC, AG_MAX_DV); else LAUNCH_W(T, TC, AG_MAX_D)
#define LAUNCH_W(T, TC, W)                                                                         \
    launch_pdl((paged_attention_generic_kernel<T, TC, W>), dim3(blocks), dim3(AG_WARPS * 32), smem, s,                      \
        static_cast<const T*>(q), static_cast<T*>(out), static_cast<const TC*>(keys),               \
        static_cast<const TC*>(values), key_page_stride, value_page_stride, positions,             \
        token_entry, entry_slot, block_table, table_stride, num_tokens, nq, nkv, d, dv, page_size, \
        window, scale, num_pages, gate, gate_stride, gate_off, out_scale, out_stride, out_off, vec, status, \
        dist_bias, dist_len, gate_per_head, rows, head_scale, log_r1, log_r2, value_row_stride, keep_first, has_sink, sink_score)
    if (dtype == LLM_DT_F32 && cache_dtype == LLM_DT_F32) { LAUNCH(float, float); }
    else if (dtype == LLM_DT_BF16 && cache_dtype == LLM_DT_BF16) { LAUNCH(bf16, bf16); }
    else if (dtype == LLM_DT_F32 && cache_dtype == LLM_DT_BF16) { LAUNCH(float, bf16); }
    else if (dtype == LLM_DT_BF16 && cache_dtype == LLM_DT_F32) { LAUNCH(bf16, float); }
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
#undef LAUNCH_W
    return launch_status();
}

// Keys and values of equal width in one tensor [pages, 2, nkv, page, d]: the values follow the keys
// inside a page.
extern "C" int llm_paged_attention_generic(
    const void* q, void* out, int dtype, const void* cache, int cache_dtype, const int32_t* positions,
    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table, int table_stride,
    int num_tokens, int nq, int nkv, int d, int page_size, int window, float scale, int num_pages,
    int32_t* status, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || (d & 15) || page_size <= 0) return LLM_REFUSED_SIZE;
    if (!aligned16(cache)) return LLM_REFUSED_ALIGN;
    const long long half = static_cast<long long>(nkv) * page_size * d;
    const char* base = static_cast<const char*>(cache);
    return llm_paged_attention_generic_kv(q, out, dtype, base, base + half * (cache_dtype == LLM_DT_F32 ? 4 : 2),
                                          cache_dtype, 2 * half, 2 * half, positions, token_entry, entry_slot,
                                          block_table, table_stride, num_tokens, nq, nkv, d, d, page_size, window,
                                          scale, num_pages, nullptr, 0, 0, 1.0f, static_cast<long long>(nq) * d, 0,
                                          status, nullptr, 0, 0, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0.0f, stream);
}
