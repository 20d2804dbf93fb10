// GPT-OSS MoE expert layer on MXFP4 weights, device-side end to end (no host round trip):
//   route (softmax, top-k, renormalise) -> count / plan / scatter tokens per expert ->
//   gather rows -> [dequantize expert group -> grouped tcgen05 GEMM + clamped SwiGLU]* ->
//   [dequantize -> grouped GEMM (down)]* -> weighted combine in ascending expert order.
// Mirrors MoeFeedForward::forward + dispatch_sparse + MoeExpert::GptOss (moe.rs:466-499,
// 563-607, 152-173); every reduction has a fixed order, so results are run-to-run identical.
#include "oxq_common.cuh"

namespace oxq {

int mxfp4_dequant_rows_bf16(const uint8_t *blocks, const uint8_t *scales, __nv_bfloat16 *out, int k, int n_off,
                            int n_cnt, cudaStream_t st);
int gemm_grouped(const void *a, int a_rows, const void *w, int slab_experts, int e_first, int nw, int k,
                 const int4 *entries, const int *grp_beg, int group, const void *bias, int bias_dtype, void *out,
                 int ldo, int epi, float limit, int *flag, cudaStream_t stream);

int moe_fused_block_rows();
bool moe_fused_supported(int n, int k, const void *blocks, const void *scales, const void *a, const void *out, int ldo);
int moe_fused_grouped(const void *a, int a_rows, const uint8_t *blocks, const uint8_t *scales, int experts, int n, int k,
                      const int4 *entries, const int *n_blocks, const void *bias, int bias_dtype, void *out, int ldo, int epi,
                      float limit, int *flag, cudaStream_t st);

bool mxfp4_gemv_batched_supported(int k, const void *blocks);
int mxfp4_gemv_batched(const void *x, int x_div, const uint8_t *blocks, const uint8_t *scales, const void *bias,
                       int bias_dtype, const int *pair_expert, int pairs, int e_lo, int e_hi, void *y, int y_dtype, int k,
                       int n, cudaStream_t st);

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_MAX_TOPK = 8;
// Up to this many (token, slot) pairs the layer runs as batched single-token GEMVs on the packed
// weights of the selected experts only (decode); above, it dequantizes expert groups for the grouped GEMM.
constexpr int MOE_DECODE_MAX_PAIRS = 64;
constexpr int MOE_DECODE_FUSED_FROM_PAIRS = 48;

// One warp per token: f32 softmax over all experts, k rounds of arg-max (ties: lower index),
// optional renormalisation by the sum of the selected probabilities (moe.rs:472-487).
__global__ void __launch_bounds__(256)
moe_route_kernel(const float *__restrict__ logits, int tokens, int experts, int top_k, int norm_topk,
                 int *__restrict__ top_idx, float *__restrict__ top_w)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= tokens) return;
    const float *l = logits + (size_t)warp * experts;
    constexpr int PER = MOE_MAX_EXPERTS / 32;
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int e = lane + 32 * i;
        v[i] = e < experts ? l[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int e = lane + 32 * i;
        v[i] = e < experts ? expf(v[i] - mx) : 0.0f;
        sum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
#pragma unroll
    for (int i = 0; i < PER; i++) v[i] = (lane + 32 * i) < experts ? v[i] / sum : -1.0f;

    float denom = 0.0f, picked_w[MOE_MAX_TOPK];
    int picked_e[MOE_MAX_TOPK];
    for (int s = 0; s < top_k; s++) {
        float best = -2.0f;
        int best_e = 0x7FFFFFFF;
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int e = lane + 32 * i;
            if (v[i] > best) { best = v[i]; best_e = e; } // increasing e within a lane: first maximum wins
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        picked_w[s] = best;
        picked_e[s] = best_e;
        denom += best;
        if ((best_e & 31) == lane) {
#pragma unroll
            for (int i = 0; i < PER; i++)
                if (lane + 32 * i == best_e) v[i] = -1.0f; // taken
        }
    }
    if (lane == 0)
        for (int s = 0; s < top_k; s++) {
            top_idx[(size_t)warp * top_k + s] = picked_e[s];
            top_w[(size_t)warp * top_k + s] = norm_topk ? picked_w[s] / denom : picked_w[s];
        }
}

// counts[e - e_lo] = number of (token, slot) pairs routed to expert e, for e in [e_lo, e_hi).
__global__ void __launch_bounds__(1024)
moe_count_kernel(const int *__restrict__ top_idx, int pairs, int e_lo, int *__restrict__ counts)
{
    __shared__ int part[32];
    const int e = e_lo + blockIdx.x;
    int c = 0;
    const int quads = pairs / 4; // top_idx sits on a 256-byte boundary of the workspace
    for (int i = threadIdx.x; i < quads; i += blockDim.x) {
        const int4 v = __ldg(reinterpret_cast<const int4 *>(top_idx) + i);
        c += (v.x == e) + (v.y == e) + (v.z == e) + (v.w == e);
    }
    for (int i = quads * 4 + threadIdx.x; i < pairs; i += blockDim.x) c += top_idx[i] == e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x < 32) {
        int t = part[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
        if (threadIdx.x == 0) counts[blockIdx.x] = t;
    }
}

// offsets = exclusive scan of counts; m-tile table (128 rows each) per expert in ascending order;
// grp_beg[g] = first m tile of expert group g (experts_per_group experts each).
__global__ void moe_plan_kernel(const int *__restrict__ counts, int n_exp, int e_lo, int experts_per_group,
                                int *__restrict__ offsets, int4 *__restrict__ entries, int *__restrict__ grp_beg)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int off = 0, mt = 0, g = 0;
    for (int i = 0; i < n_exp; i++) {
        if (i % experts_per_group == 0) grp_beg[g++] = mt;
        offsets[i] = off;
        const int c = counts[i];
        for (int r = 0; r < c; r += 128) entries[mt++] = make_int4(off + r, min(128, c - r), e_lo + i, 0);
        off += c;
    }
    offsets[n_exp] = off;
    grp_beg[g] = mt;
}

// The same offsets; token blocks for the kernel that unpacks MXFP4 inside the tensor-core loop: every expert's rows cut into
// the fewest blocks of at most max_rows rows, of equal size rounded up to 16. n_blocks[0] = how many.
__global__ void moe_plan_blocks_kernel(const int *__restrict__ counts, int n_exp, int e_lo, int max_rows, int *__restrict__ offsets,
                                       int4 *__restrict__ entries, int *__restrict__ n_blocks)
{
    __shared__ int cnt_s[MOE_MAX_EXPERTS];
    for (int i = threadIdx.x; i < n_exp; i += blockDim.x) cnt_s[i] = counts[i]; // one round trip for all counts
    __syncthreads();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int off = 0, nb = 0;
    for (int i = 0; i < n_exp; i++) {
        offsets[i] = off;
        const int c = cnt_s[i];
        if (c > 0) {
            const int parts = (c + max_rows - 1) / max_rows;
            const int size = ((c + parts - 1) / parts + 15) / 16 * 16;
            for (int r = 0; r < c; r += size) entries[nb++] = make_int4(off + r, min(size, c - r), e_lo + i, 0);
        }
        off += c;
    }
    offsets[n_exp] = off;
    n_blocks[0] = nb;
}

// Stable partition: position of pair i among the pairs of its expert, in pair (= token) order.
// One CTA per expert walks the pairs 4096 at a time (four neighbours per thread); a scan over the threads'
// hit counts keeps the order deterministic.
__global__ void __launch_bounds__(1024)
moe_scatter_kernel(const int *__restrict__ top_idx, int pairs, int e_lo, const int *__restrict__ offsets,
                   int *__restrict__ perm, int *__restrict__ inv)
{
    __shared__ int warp_cnt[32], warp_off[32];
    __shared__ int total_s;
    const int e = e_lo + blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int base = offsets[blockIdx.x];
    for (int start = 0; start < pairs; start += 4096) {
        const int i0 = start + 4 * (int)threadIdx.x;
        int id[4] = {-1, -1, -1, -1};
        if (i0 + 3 < pairs) {
            const int4 v = __ldg(reinterpret_cast<const int4 *>(top_idx + i0)); // top_idx sits on a 256-byte boundary
            id[0] = v.x; id[1] = v.y; id[2] = v.z; id[3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (i0 + j < pairs) id[j] = top_idx[i0 + j];
        }
        const int cnt = (id[0] == e) + (id[1] == e) + (id[2] == e) + (id[3] == e);
        int incl = cnt; // inclusive scan of the hit counts over the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_cnt[warp] = incl;
        __syncthreads();
        if (warp == 0) { // exclusive scan of the warps' totals
            const int c = warp_cnt[lane];
            int inc2 = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xFFFFFFFFu, inc2, o);
                if (lane >= o) inc2 += t;
            }
            warp_off[lane] = inc2 - c;
            if (lane == 31) total_s = inc2;
        }
        __syncthreads();
        int pos = base + warp_off[warp] + incl - cnt;
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (id[j] == e) {
                perm[pos] = i0 + j;
                inv[i0 + j] = pos;
                pos += 1;
            }
        base += total_s;
        __syncthreads(); // warp_cnt, warp_off and total_s are rewritten by the next pass
    }
}

// xs[pos, :] = x[perm[pos] / top_k, :]  (one warp per row, 16-byte copies)
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16 *__restrict__ x, const int *__restrict__ perm, const int *__restrict__ total_rows,
                  int top_k, int hidden, __nv_bfloat16 *__restrict__ xs, int rows_by_value = 0)
{
    const int rows = total_rows ? *total_rows : rows_by_value;
    const int lane = threadIdx.x & 31;
    for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += (gridDim.x * blockDim.x) >> 5) {
        const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)(perm[row] / top_k) * hidden);
        uint4 *dst = reinterpret_cast<uint4 *>(xs + (size_t)row * hidden);
        for (int c = lane; c < hidden / 8; c += 32) dst[c] = src[c];
    }
}

// out[t, :] = sum over the token's slots whose expert is in [e_lo, e_hi), in ascending expert id,
// of w * yp[inv[pair], :] (f32 accumulation, one rounding). Tokens without such a slot get zeros.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16 *__restrict__ yp, const int *__restrict__ top_idx, const float *__restrict__ top_w,
                   const int *__restrict__ inv, int tokens, int top_k, int hidden, int e_lo, int e_hi, void *out,
                   int out_dtype)
{
    const int chunks = hidden / 8;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < (size_t)tokens * chunks;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / chunks), c = (int)(idx % chunks);
        int order[MOE_MAX_TOPK], ids[MOE_MAX_TOPK];
#pragma unroll
        for (int s = 0; s < MOE_MAX_TOPK; s++) {
            order[s] = s;
            ids[s] = s < top_k ? __ldg(top_idx + (size_t)t * top_k + s) : 0x7FFFFFFF;
        }
#pragma unroll
        for (int a = 1; a < MOE_MAX_TOPK; a++) // insertion sort by expert id (k <= 8), in registers
#pragma unroll
            for (int b = a; b > 0; b--)
                if (ids[b] < ids[b - 1]) {
                    const int ti = ids[b]; ids[b] = ids[b - 1]; ids[b - 1] = ti;
                    const int to = order[b]; order[b] = order[b - 1]; order[b - 1] = to;
                }
        // all index loads first, then all row loads, then the sums in ascending expert order: the loads of a token's
        // slots do not wait for one another
        int pos[MOE_MAX_TOPK];
        float wv[MOE_MAX_TOPK];
        bool use[MOE_MAX_TOPK];
#pragma unroll
        for (int s = 0; s < MOE_MAX_TOPK; s++) {
            use[s] = s < top_k && ids[s] >= e_lo && ids[s] < e_hi;
            const size_t pair = (size_t)t * top_k + order[s];
            pos[s] = use[s] ? __ldg(inv + pair) : 0;
            wv[s] = use[s] ? __ldg(top_w + pair) : 0.0f;
        }
        uint4 rows[MOE_MAX_TOPK];
#pragma unroll
        for (int s = 0; s < MOE_MAX_TOPK; s++)
            rows[s] = use[s] ? reinterpret_cast<const uint4 *>(yp + (size_t)pos[s] * hidden)[c] : make_uint4(0u, 0u, 0u, 0u);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int s = 0; s < MOE_MAX_TOPK; s++) {
            if (!use[s]) continue;
            const float w = wv[s];
            const uint32_t vv[4] = {rows[s].x, rows[s].y, rows[s].z, rows[s].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                acc[2 * q] = fmaf(w, __uint_as_float(vv[q] << 16), acc[2 * q]);
                acc[2 * q + 1] = fmaf(w, __uint_as_float(vv[q] & 0xFFFF0000u), acc[2 * q + 1]);
            }
        }
        for (int q = 0; q < 8; q++) store_as(out, out_dtype, (size_t)t * hidden + c * 8 + q, acc[q]);
    }
}

// Decode path: h[pair, j] = clamped SwiGLU of the interleaved (gate, up) columns 2j, 2j+1 of gu[pair, :]
// (moe.rs:152-173; the same arithmetic as the grouped GEMM's epilogue), and inv[pair] = pair.
__global__ void __launch_bounds__(256)
moe_swiglu_kernel(const float *__restrict__ gu, int pairs, int inter, float limit, __nv_bfloat16 *__restrict__ h,
                  int *__restrict__ inv)
{
    const size_t total = (size_t)pairs * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const float2 v = reinterpret_cast<const float2 *>(gu)[idx];
        const float gate = fminf(v.x, limit), up = fminf(fmaxf(v.y, -limit), limit);
        const float sig = __fdividef(1.0f, __expf(-1.702f * gate) + 1.0f);
        h[idx] = __float2bfloat16_rn((up + 1.0f) * (gate * sig));
        if (idx < (size_t)pairs) inv[idx] = (int)idx;
    }
}

// offsets = exclusive scan of counts (one warp; at most MOE_MAX_EXPERTS entries).
__global__ void moe_offsets_kernel(const int *__restrict__ counts, int n, int *__restrict__ offsets)
{
    __shared__ int cnt_s[MOE_MAX_EXPERTS];
    for (int i = threadIdx.x; i < n; i += blockDim.x) cnt_s[i] = counts[i];
    __syncthreads();
    if (threadIdx.x != 0) return;
    int off = 0;
    for (int i = 0; i < n; i++) { offsets[i] = off; off += cnt_s[i]; }
    offsets[n] = off;
}

// ids of rows that arrive grouped: group g (source rank g / n_local, local expert g % n_local) holds counts[g] rows of
// expert lo + g % n_local. One CTA: scan of the group sizes in shared memory, then every thread fills whole groups.
__global__ void __launch_bounds__(1024)
moe_expand_ids_kernel(const int *__restrict__ counts, int groups, int n_local, int lo, int *__restrict__ ids)
{
    __shared__ int start_s[2049];
    if (threadIdx.x == 0) {
        int off = 0;
        for (int g = 0; g < groups; g++) { start_s[g] = off; off += counts[g]; }
        start_s[groups] = off;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = warp; g < groups; g += 32) {
        const int a = start_s[g], b = start_s[g + 1], e = lo + g % n_local;
        for (int i = a + lane; i < b; i += 32) ids[i] = e;
    }
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct MoeLayout {
    size_t top_idx, top_w, counts, offsets, grp_beg, entries, perm, inv, xs, h, slab, total;
    int group_experts, n_groups, max_mt;
    bool decode; // few pairs: no dequantized slab, the slab region holds the f32 gate_up outputs
};

static bool moe_decode_shape(size_t pairs, int hidden, int inter)
{
    return pairs <= (size_t)MOE_DECODE_MAX_PAIRS && hidden % 32 == 0 && inter % 32 == 0 &&
           mxfp4_gemv_batched_supported(hidden, nullptr) && mxfp4_gemv_batched_supported(inter, nullptr);
}

static MoeLayout moe_layout(int tokens, int top_k, int n_exp, int hidden, int inter)
{
    MoeLayout L;
    const size_t pairs = (size_t)tokens * top_k;
    // Experts dequantized at once: as many as fit 1152 MiB of bf16 gate_up weights (all 32 experts of
    // a GPT-OSS-20B layer), at least one. One grouped GEMM over many experts fills whole rounds of
    // the persistent grid; small groups left a third of the SM-rounds idle and paid a launch each.
    const size_t per_expert = (size_t)2 * inter * hidden * 2;
    int ge = (int)(((size_t)1152 << 20) / per_expert);
    if (ge < 1) ge = 1;
    if (ge > n_exp) ge = n_exp;
    L.group_experts = ge;
    L.n_groups = (n_exp + ge - 1) / ge;
    L.max_mt = (int)(pairs / 128) + n_exp + 1;
    size_t off = 256;
    L.top_idx = off; off = align_up(off + pairs * 4, 256);
    L.top_w = off; off = align_up(off + pairs * 4, 256);
    L.counts = off; off = align_up(off + (size_t)n_exp * 4, 256);
    L.offsets = off; off = align_up(off + (size_t)(n_exp + 1) * 4, 256);
    L.grp_beg = off; off = align_up(off + (size_t)(L.n_groups + 1) * 4, 256);
    L.entries = off; off = align_up(off + (size_t)L.max_mt * 16, 256);
    L.perm = off; off = align_up(off + pairs * 4, 256);
    L.inv = off; off = align_up(off + pairs * 4, 256);
    L.xs = off; off = align_up(off + (pairs + 128) * hidden * 2, 256); // also the down-projection output
    L.h = off; off = align_up(off + (pairs + 128) * inter * 2, 256);
    L.decode = moe_decode_shape(pairs, hidden, inter);
    L.slab = off; off = align_up(off + (L.decode ? pairs * 2 * inter * sizeof(float) : (size_t)ge * per_expert), 256);
    L.total = off;
    return L;
}

} // namespace oxq

using namespace oxq;

OXQ_EXPORT size_t oxq_gptoss_moe_workspace_bytes(int tokens, int top_k, int num_local_experts, int hidden, int inter)
{
    if (tokens <= 0 || top_k <= 0 || num_local_experts <= 0 || hidden <= 0 || inter <= 0) return 0;
    return moe_layout(tokens, top_k, num_local_experts, hidden, inter).total;
}

// Rows that already carry their expert: top_idx = the given id, weight one (the owner side of expert parallelism).
__global__ void __launch_bounds__(256) moe_assign_kernel(const int32_t *__restrict__ ids, int rows, int *__restrict__ top_idx,
                                                         float *__restrict__ top_w)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) { top_idx[i] = ids[i]; top_w[i] = 1.0f; }
}

static int moe_forward_impl(const void *x, int x_dtype, const float *router_logits, const int32_t *given_ids, int tokens,
                            int num_experts, int top_k, int norm_topk, int hidden, int inter, const uint8_t *gu_blocks,
                            const uint8_t *gu_scales, const void *gu_bias, const uint8_t *dn_blocks,
                            const uint8_t *dn_scales, const void *dn_bias, int bias_dtype, float limit,
                            int expert_lo, int expert_hi, void *out, int out_dtype, void *workspace,
                            size_t workspace_bytes, void *stream)
{
    OXQ_REQUIRE(x && (router_logits || given_ids) && gu_blocks && gu_scales && dn_blocks && dn_scales && out, OXQ_ERR_NULL,
                "oxq_gptoss_moe_forward: null pointer");
    OXQ_REQUIRE(x_dtype == OXQ_BF16, OXQ_ERR_UNSUPPORTED, "oxq_gptoss_moe_forward: activations must be bf16");
    OXQ_REQUIRE(valid_dtype(out_dtype) && (!(gu_bias || dn_bias) || valid_dtype(bias_dtype)), OXQ_ERR_UNSUPPORTED,
                "oxq_gptoss_moe_forward: unsupported dtype");
    OXQ_REQUIRE(tokens > 0 && num_experts > 0 && num_experts <= MOE_MAX_EXPERTS && top_k > 0 && top_k <= MOE_MAX_TOPK &&
                    top_k <= num_experts,
                OXQ_ERR_BAD_SHAPE, "oxq_gptoss_moe_forward: tokens %d, experts %d (max %d), top_k %d (max %d)", tokens,
                num_experts, MOE_MAX_EXPERTS, top_k, MOE_MAX_TOPK);
    OXQ_REQUIRE(hidden % 32 == 0 && inter % 32 == 0, OXQ_ERR_BAD_SHAPE,
                "Mxfp4Linear: in_features (%d, %d) must be a multiple of 32", hidden, inter);
    OXQ_REQUIRE(0 <= expert_lo && expert_lo < expert_hi && expert_hi <= num_experts, OXQ_ERR_BAD_SHAPE,
                "oxq_gptoss_moe_forward: expert range [%d, %d) outside 0..%d", expert_lo, expert_hi, num_experts);
    const int n_exp = expert_hi - expert_lo;
    const MoeLayout L = moe_layout(tokens, top_k, n_exp, hidden, inter);
    OXQ_REQUIRE(workspace && workspace_bytes >= L.total, OXQ_ERR_WORKSPACE,
                "oxq_gptoss_moe_forward: workspace of %zu bytes needed, got %zu", L.total, workspace_bytes);
    OXQ_REQUIRE(aligned(workspace, 256) && aligned(x, 16), OXQ_ERR_BAD_ALIGN,
                "oxq_gptoss_moe_forward: workspace must be 256-byte and x 16-byte aligned");

    cudaStream_t st = (cudaStream_t)stream;
    unsigned char *ws = reinterpret_cast<unsigned char *>(workspace);
    int *flag = reinterpret_cast<int *>(ws);
    int *top_idx = reinterpret_cast<int *>(ws + L.top_idx);
    float *top_w = reinterpret_cast<float *>(ws + L.top_w);
    int *counts = reinterpret_cast<int *>(ws + L.counts), *offsets = reinterpret_cast<int *>(ws + L.offsets);
    int *grp_beg = reinterpret_cast<int *>(ws + L.grp_beg);
    int4 *entries = reinterpret_cast<int4 *>(ws + L.entries);
    int *perm = reinterpret_cast<int *>(ws + L.perm), *inv = reinterpret_cast<int *>(ws + L.inv);
    __nv_bfloat16 *xs = reinterpret_cast<__nv_bfloat16 *>(ws + L.xs), *h = reinterpret_cast<__nv_bfloat16 *>(ws + L.h);
    __nv_bfloat16 *slab = reinterpret_cast<__nv_bfloat16 *>(ws + L.slab);
    const int pairs = tokens * top_k;

    if (given_ids) moe_assign_kernel<<<ceil_div(tokens, 256), 256, 0, st>>>(given_ids, tokens, top_idx, top_w);
    else moe_route_kernel<<<ceil_div(tokens * 32, 256), 256, 0, st>>>(router_logits, tokens, num_experts, top_k, norm_topk,
                                                                      top_idx, top_w);
    const int a_rows = pairs + 128;
    // Both projections through the kernel that unpacks the MXFP4 blocks inside the tensor-core loop, where it takes the shapes:
    // no dequantized slab, one launch per projection over all experts.
    const bool fused = moe_fused_supported(2 * inter, hidden, gu_blocks, gu_scales, xs, h, inter) &&
                       moe_fused_supported(hidden, inter, dn_blocks, dn_scales, h, xs, hidden);
    // The per-pair GEMVs cost about 6.3 us a pair on the GPT-OSS shape (201 us at 32 pairs); the grouped kernel reads every
    // expert that has rows once, 0.32 ms at 128 pairs: it takes over from about 48 pairs.
    if (L.decode && !(fused && pairs > MOE_DECODE_FUSED_FROM_PAIRS)) {
        OXQ_REQUIRE(aligned(gu_blocks, 16) && aligned(dn_blocks, 16), OXQ_ERR_BAD_ALIGN,
                    "oxq_gptoss_moe_forward: expert blocks must be 16-byte aligned");
        // Decode: only the selected experts' packed weights are read. gate_up (f32 out, bias folded) ->
        // SwiGLU -> down (into the xs buffer, bf16) -> combine with inv = identity.
        OXQ_LAUNCH_CHECK("moe_route_kernel");
        float *gu = reinterpret_cast<float *>(slab);
        int rc = mxfp4_gemv_batched(x, top_k, gu_blocks, gu_scales, gu_bias, bias_dtype, top_idx, pairs, expert_lo, expert_hi,
                                    gu, OXQ_F32, hidden, 2 * inter, st);
        if (rc) return rc;
        moe_swiglu_kernel<<<ceil_div(pairs * inter, 256), 256, 0, st>>>(gu, pairs, inter, limit, h, inv);
        OXQ_LAUNCH_CHECK("moe_swiglu_kernel");
        rc = mxfp4_gemv_batched(h, 1, dn_blocks, dn_scales, dn_bias, bias_dtype, top_idx, pairs, expert_lo, expert_hi, xs,
                                OXQ_BF16, inter, hidden, st);
        if (rc) return rc;
        moe_combine_kernel<<<ceil_div(tokens * (hidden / 8), 256), 256, 0, st>>>(xs, top_idx, top_w, inv, tokens, top_k,
                                                                                 hidden, expert_lo, expert_hi, out, out_dtype);
        OXQ_LAUNCH_CHECK("moe_combine_kernel");
        return OXQ_OK;
    }
    moe_count_kernel<<<n_exp, 1024, 0, st>>>(top_idx, pairs, expert_lo, counts);
    // the grouped kernel's table of token blocks goes where the m-tile table of the dense path would (same capacity bound);
    // grp_beg[0] then holds the number of blocks
    if (fused) moe_plan_blocks_kernel<<<1, 32, 0, st>>>(counts, n_exp, expert_lo, moe_fused_block_rows(), offsets, entries, grp_beg);
    else moe_plan_kernel<<<1, 32, 0, st>>>(counts, n_exp, expert_lo, L.group_experts, offsets, entries, grp_beg);
    moe_scatter_kernel<<<n_exp, 1024, 0, st>>>(top_idx, pairs, expert_lo, offsets, perm, inv);
    moe_gather_kernel<<<sm_count() * 8, 256, 0, st>>>((const __nv_bfloat16 *)x, perm, offsets + n_exp, top_k, hidden, xs);
    OXQ_LAUNCH_CHECK("moe routing kernels");

    if (fused) {
        int rc = moe_fused_grouped(xs, a_rows, gu_blocks, gu_scales, num_experts, 2 * inter, hidden, entries, grp_beg, gu_bias,
                                   bias_dtype, h, inter, 1, limit, flag, st);
        if (rc) return rc;
        rc = moe_fused_grouped(h, a_rows, dn_blocks, dn_scales, num_experts, hidden, inter, entries, grp_beg, dn_bias, bias_dtype,
                               xs, hidden, 0, limit, flag, st);
        if (rc) return rc;
        moe_combine_kernel<<<sm_count() * 8, 256, 0, st>>>(xs, top_idx, top_w, inv, tokens, top_k, hidden, expert_lo, expert_hi,
                                                         out, out_dtype);
        OXQ_LAUNCH_CHECK("moe_combine_kernel");
        return OXQ_OK;
    }
    const size_t gu_rows = (size_t)2 * inter, nbh = hidden / 32, nbi = inter / 32;
    for (int g = 0; g < L.n_groups; g++) { // gate_up + SwiGLU: h = act(xs . W_gu^T + b_gu)
        const int e0 = expert_lo + g * L.group_experts;
        const int ne = (e0 + L.group_experts <= expert_hi) ? L.group_experts : expert_hi - e0;
        int rc = mxfp4_dequant_rows_bf16(gu_blocks + (size_t)e0 * gu_rows * nbh * 16, gu_scales + (size_t)e0 * gu_rows * nbh,
                                         slab, hidden, 0, (int)(ne * gu_rows), st);
        if (rc) return rc;
        rc = gemm_grouped(xs, a_rows, slab, ne, e0, (int)gu_rows, hidden, entries, grp_beg, g, gu_bias, bias_dtype, h,
                          inter, 1, limit, flag, st);
        if (rc) return rc;
    }
    for (int g = 0; g < L.n_groups; g++) { // down: yp = h . W_dn^T + b_dn (into the xs buffer)
        const int e0 = expert_lo + g * L.group_experts;
        const int ne = (e0 + L.group_experts <= expert_hi) ? L.group_experts : expert_hi - e0;
        int rc = mxfp4_dequant_rows_bf16(dn_blocks + (size_t)e0 * hidden * nbi * 16, dn_scales + (size_t)e0 * hidden * nbi,
                                         slab, inter, 0, ne * hidden, st);
        if (rc) return rc;
        rc = gemm_grouped(h, a_rows, slab, ne, e0, hidden, inter, entries, grp_beg, g, dn_bias, bias_dtype, xs, hidden,
                          0, limit, flag, st);
        if (rc) return rc;
    }
    moe_combine_kernel<<<sm_count() * 8, 256, 0, st>>>(xs, top_idx, top_w, inv, tokens, top_k, hidden, expert_lo, expert_hi, out,
                                                out_dtype);
    OXQ_LAUNCH_CHECK("moe_combine_kernel");
    return OXQ_OK;
}

OXQ_EXPORT int oxq_gptoss_moe_forward(const void *x, int x_dtype, const float *router_logits, int tokens, int num_experts,
                                      int top_k, int norm_topk, int hidden, int inter, const uint8_t *gu_blocks,
                                      const uint8_t *gu_scales, const void *gu_bias, const uint8_t *dn_blocks,
                                      const uint8_t *dn_scales, const void *dn_bias, int bias_dtype, float limit,
                                      int expert_lo, int expert_hi, void *out, int out_dtype, void *workspace,
                                      size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(router_logits != nullptr, OXQ_ERR_NULL, "oxq_gptoss_moe_forward: null pointer");
    return moe_forward_impl(x, x_dtype, router_logits, nullptr, tokens, num_experts, top_k, norm_topk, hidden, inter, gu_blocks,
                            gu_scales, gu_bias, dn_blocks, dn_scales, dn_bias, bias_dtype, limit, expert_lo, expert_hi, out,
                            out_dtype, workspace, workspace_bytes, stream);
}

// Each row through the expert it is already assigned to, weight one: out[r] = expert[ids[r]](rows[r]).
OXQ_EXPORT int oxq_gptoss_experts_forward(const void *rows, int x_dtype, const int32_t *expert_ids, int n_rows, int num_experts,
                                          int hidden, int inter, const uint8_t *gu_blocks, const uint8_t *gu_scales,
                                          const void *gu_bias, const uint8_t *dn_blocks, const uint8_t *dn_scales,
                                          const void *dn_bias, int bias_dtype, float limit, int expert_lo, int expert_hi,
                                          void *out, int out_dtype, void *workspace, size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(expert_ids != nullptr, OXQ_ERR_NULL, "oxq_gptoss_experts_forward: null pointer");
    return moe_forward_impl(rows, x_dtype, nullptr, expert_ids, n_rows, num_experts, 1, 0, hidden, inter, gu_blocks, gu_scales,
                            gu_bias, dn_blocks, dn_scales, dn_bias, bias_dtype, limit, expert_lo, expert_hi, out, out_dtype,
                            workspace, workspace_bytes, stream);
}

// Weighted sum of each token's k result rows in ascending expert order (moe.rs:593-605: index_add per expert in order):
// out[t] = sum_s top_w[t, s] * rows[pos[t * k + s]]; f32 accumulation, one rounding. Same bits every run.
OXQ_EXPORT int oxq_moe_combine(const void *rows, const int32_t *top_idx, const float *top_w, const int32_t *pos, int tokens,
                               int top_k, int hidden, int num_experts, void *out, int out_dtype, void *stream)
{
    clear_error();
    OXQ_REQUIRE(rows && top_idx && top_w && pos && out, OXQ_ERR_NULL, "oxq_moe_combine: null pointer");
    OXQ_REQUIRE(valid_dtype(out_dtype), OXQ_ERR_UNSUPPORTED, "oxq_moe_combine: unsupported dtype");
    OXQ_REQUIRE(tokens > 0 && top_k > 0 && top_k <= MOE_MAX_TOPK && hidden > 0 && hidden % 8 == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_moe_combine: tokens %d, top_k %d (max %d), hidden %d (multiple of 8)", tokens, top_k, MOE_MAX_TOPK, hidden);
    OXQ_REQUIRE(aligned(rows, 16), OXQ_ERR_BAD_ALIGN, "oxq_moe_combine: rows must be 16-byte aligned");
    moe_combine_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)rows, top_idx, top_w, pos, tokens,
                                                                          top_k, hidden, 0, num_experts, out, out_dtype);
    OXQ_LAUNCH_CHECK("moe_combine_kernel");
    return OXQ_OK;
}

// Routing alone (moe.rs:472-487): top_idx i32 [tokens, top_k], top_w f32 [tokens, top_k].
OXQ_EXPORT int oxq_moe_route(const float *router_logits, int tokens, int num_experts, int top_k, int norm_topk,
                             int32_t *top_idx, float *top_w, void *stream)
{
    clear_error();
    OXQ_REQUIRE(router_logits && top_idx && top_w, OXQ_ERR_NULL, "oxq_moe_route: null pointer");
    OXQ_REQUIRE(tokens > 0 && num_experts > 0 && num_experts <= MOE_MAX_EXPERTS && top_k > 0 && top_k <= MOE_MAX_TOPK &&
                    top_k <= num_experts,
                OXQ_ERR_BAD_SHAPE, "oxq_moe_route: tokens %d, experts %d (max %d), top_k %d (max %d)", tokens, num_experts,
                MOE_MAX_EXPERTS, top_k, MOE_MAX_TOPK);
    moe_route_kernel<<<ceil_div(tokens * 32, 256), 256, 0, (cudaStream_t)stream>>>(router_logits, tokens, num_experts,
                                                                                    top_k, norm_topk, top_idx, top_w);
    OXQ_LAUNCH_CHECK("moe_route_kernel");
    return OXQ_OK;
}

// Dispatch plan of expert parallelism on the device (the sender side of dispatch_sparse, moe.rs:563-607, when experts live on
// other ranks): pairs (token, slot) sorted by expert id, pair order kept inside an expert. counts [E], offsets [E + 1],
// perm [pairs] (perm[i] = pair sent i-th), inv [pairs] (inv[pair] = its position). No counterpart in the reference.
OXQ_EXPORT int oxq_moe_dispatch_plan(const int32_t *top_idx, int pairs, int num_experts, int32_t *counts, int32_t *offsets,
                                     int32_t *perm, int32_t *inv, void *stream)
{
    clear_error();
    OXQ_REQUIRE(top_idx && counts && offsets && perm && inv, OXQ_ERR_NULL, "oxq_moe_dispatch_plan: null pointer");
    OXQ_REQUIRE(pairs > 0 && num_experts > 0 && num_experts <= MOE_MAX_EXPERTS, OXQ_ERR_BAD_SHAPE,
                "oxq_moe_dispatch_plan: pairs %d, experts %d (max %d)", pairs, num_experts, MOE_MAX_EXPERTS);
    OXQ_REQUIRE(aligned(top_idx, 16), OXQ_ERR_BAD_ALIGN, "oxq_moe_dispatch_plan: top_idx must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    moe_count_kernel<<<num_experts, 1024, 0, st>>>(top_idx, pairs, 0, counts);
    moe_offsets_kernel<<<1, 32, 0, st>>>(counts, num_experts, offsets);
    moe_scatter_kernel<<<num_experts, 1024, 0, st>>>(top_idx, pairs, 0, offsets, perm, inv);
    OXQ_LAUNCH_CHECK("moe dispatch plan kernels");
    return OXQ_OK;
}

// out[i, :] = x[perm[i] / top_k, :] for i < rows (bf16 rows, hidden a multiple of 8): the rows of a dispatch in send order.
OXQ_EXPORT int oxq_moe_gather_rows(const void *x, const int32_t *perm, int rows, int top_k, int hidden, void *out, void *stream)
{
    clear_error();
    OXQ_REQUIRE(x && perm && out, OXQ_ERR_NULL, "oxq_moe_gather_rows: null pointer");
    OXQ_REQUIRE(rows > 0 && top_k > 0 && hidden > 0 && hidden % 8 == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_moe_gather_rows: rows %d, top_k %d, hidden %d (multiple of 8)", rows, top_k, hidden);
    OXQ_REQUIRE(aligned(x, 16) && aligned(out, 16), OXQ_ERR_BAD_ALIGN, "oxq_moe_gather_rows: rows must be 16-byte aligned");
    moe_gather_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)x, perm, nullptr, top_k, hidden,
                                                                         (__nv_bfloat16 *)out, rows);
    OXQ_LAUNCH_CHECK("moe_gather_kernel");
    return OXQ_OK;
}

// Expert ids of rows received in groups (source rank major, local expert minor): counts [world * n_local] -> ids [total].
OXQ_EXPORT int oxq_moe_expand_ids(const int32_t *counts, int groups, int n_local, int lo, int32_t *ids, void *stream)
{
    clear_error();
    OXQ_REQUIRE(counts && ids, OXQ_ERR_NULL, "oxq_moe_expand_ids: null pointer");
    OXQ_REQUIRE(groups > 0 && groups <= 2048 && n_local > 0 && groups % n_local == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_moe_expand_ids: groups %d (at most 2048, a multiple of n_local %d)", groups, n_local);
    moe_expand_ids_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(counts, groups, n_local, lo, ids);
    OXQ_LAUNCH_CHECK("moe_expand_ids_kernel");
    return OXQ_OK;
}
