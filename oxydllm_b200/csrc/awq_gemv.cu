// AWQ W4A16 batched decode GEMV, 1 <= m <= 32. Two kernels:
//
//  * awq_gemv_group_kernel (second half of this file) is the one the operator
//    launches whenever group_size is a power of two >= 16 and the shape tiles
//    (every benchmark layer): k slices aligned to quantization groups, packed
//    words streamed from HBM straight into registers a few steps ahead, x staged
//    once per CTA in shared memory as f16, nibbles turned into exact f16 values
//    with one lop3 each, mma.sync m16n8k16 f16 with f32 accumulation, scale and
//    zero point folded once per group in f32, split-k partials summed in fixed
//    order through (distributed) shared memory of a thread-block cluster. Its
//    own comment below has the details.
//  * awq_gemv_kernel (first half) is the general fallback for the remaining
//    shapes (odd group sizes, k not a multiple of the slice): every lane copies
//    the packed words it will consume with cp.async into a lane-private slot of
//    a shared-memory ring (GEMV_STAGES deep, no barrier between producer and
//    consumer); a warp step covers 16 input rows x 8V packed words; nibbles
//    become bf16 pairs along k with one prmt + one lop3 per weight
//    (0x4300 | q == 128 + q exactly) and meet up to 8 tokens in mma.sync
//    m16n8k16 bf16; one extra MMA against an all-ones operand yields sum_k x
//    per token, so  y += s * (sum (128+q) x - (128+z) sum x)  per group in f32;
//    the split along k is reduced in fixed rank order through distributed
//    shared memory: no workspace, no second launch, no atomics.
//
// Both are bound by the stream of packed weights from HBM (0.5 B per weight
// plus scales and zeros); neither allocates or synchronises.
#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>

#include "oxq_common.cuh"
#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace oxq {

constexpr int GEMV_STAGES = 8;

#ifdef OXQ_TUNING
__device__ unsigned long long g_gv_cta[1024][8]; // per-CTA time stamps of the last launch (tuning builds only)
#define GV_CTA(slot) do { if (threadIdx.x == 0) { const unsigned b_ = blockIdx.y * gridDim.x + blockIdx.x; if (b_ < 1024) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_gv_cta[b_][slot] = t_; } } } while (0)
#else
#define GV_CTA(slot) do { } while (0)
#endif

struct AwqGemvParams {
    const __nv_bfloat16 *x;
    const uint32_t *qweight;
    const uint32_t *qzeros;
    const void *scales;
    const void *bias;
    void *y;
    int scales_dtype, bias_dtype, y_dtype;
    int m, k, n, group_size;
    int packed_out;
    int steps_per_cta; // 16-row steps handled by one CTA of the cluster
    int stages;        // TMA variant: depth of a warp's ring of weight boxes
    int token_split;   // main variant: neighbouring CTAs that share an n tile and take 8*MT tokens each (>= 1)
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int BYTES> __device__ __forceinline__ void cp_async(uint32_t smem_addr, const void *gptr, bool valid)
{
    const uint32_t src_size = valid ? BYTES : 0; // 0 -> the slot is zero-filled, the source is not read
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;\n" ::"r"(smem_addr), "l"(gptr), "n"(BYTES),
                 "r"(src_size)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Nibble `slot` (0..7) of w0 and of w1 as the bf16 pair (128 + q0, 128 + q1).
// Slots 2b and 2b+1 live in byte b: gather byte b of both words with one prmt.
template <int B> __device__ __forceinline__ uint32_t gather_byte(uint32_t w0, uint32_t w1)
{
    return __byte_perm(w0, w1, B | (B << 4) | ((4 + B) << 8) | ((4 + B) << 12));
}
__device__ __forceinline__ uint32_t lo_nibbles_bf16(uint32_t p) { return (p & 0x000F000Fu) | 0x43004300u; }
__device__ __forceinline__ uint32_t hi_nibbles_bf16(uint32_t p) { return ((p >> 4) & 0x000F000Fu) | 0x43004300u; }

// MT: 8-token tiles (m <= 8*MT). V: packed words per lane per input row.
template <int MT, int V, int NW>
__global__ void __launch_bounds__(NW * 32, 1) awq_gemv_kernel(const AwqGemvParams p)
{
    constexpr int NT = NW * 32;
    constexpr int NACC = V * 4 * MT * 4;
    constexpr int W_BYTES = 4 * V;                            // per lane per row
    constexpr int STAGE_BYTES = 32 * (4 * W_BYTES + 8 * MT);  // per warp
    extern __shared__ __align__(16) unsigned char smem[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, c = lane & 3;
    const int rank = blockIdx.y, nranks = gridDim.y;

    const int jbase = (blockIdx.x * NW + warp) * 8 * V + g * V; // first packed word of this lane
    const bool j_ok = jbase < p.packed_out;                     // packed_out % V == 0: all or nothing
    const int total_steps = p.k >> 4;
    const int step_beg = rank * p.steps_per_cta;
    const int step_end = min(total_steps, step_beg + p.steps_per_cta);
    const int steps = max(0, step_end - step_beg);

    unsigned char *ring = smem + (size_t)warp * GEMV_STAGES * STAGE_BYTES;
    const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring);
    // slot layout per stage: [row i][lane] W_BYTES, then [mt][lane] 8 bytes of x
    const uint32_t w_off = lane * W_BYTES, x_off = 4 * 32 * W_BYTES + lane * 8;

    auto issue = [&](int s) {
        const uint32_t base = ring_addr + (uint32_t)(s % GEMV_STAGES) * STAGE_BYTES;
        const int kb = (step_beg + s) * 16 + 4 * c;
        const uint32_t *wsrc = p.qweight + (size_t)kb * p.packed_out + (j_ok ? jbase : 0);
#pragma unroll
        for (int i = 0; i < 4; i++)
            cp_async<W_BYTES>(base + i * 32 * W_BYTES + w_off, wsrc + (size_t)i * p.packed_out, j_ok);
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int row = 8 * mt + g;
            const bool ok = row < p.m;
            cp_async<8>(base + x_off + mt * 32 * 8, p.x + (size_t)(ok ? row : 0) * p.k + kb, ok);
        }
    };

    float acc[V][4][MT][4], tot[V][4][MT][4], sx[MT][4];
#pragma unroll
    for (int v = 0; v < V; v++)
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[v][t][mt][e] = tot[v][t][mt][e] = 0.0f;
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) sx[mt][e] = 0.0f;

#pragma unroll
    for (int s = 0; s < GEMV_STAGES - 1; s++) {
        if (s < steps) issue(s);
        cp_async_commit();
    }

    const uint32_t ones[4] = {0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u};

    for (int s = 0; s < steps; s++) {
        cp_async_wait<GEMV_STAGES - 2>();
        if (s + GEMV_STAGES - 1 < steps) issue(s + GEMV_STAGES - 1);
        cp_async_commit();

        const unsigned char *st = ring + (size_t)(s % GEMV_STAGES) * STAGE_BYTES;
        uint32_t w[4][V], xb[MT][2];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (V == 1) w[i][0] = *reinterpret_cast<const uint32_t *>(st + i * 32 * W_BYTES + w_off);
            else if (V == 2) {
                const uint2 t2 = *reinterpret_cast<const uint2 *>(st + i * 32 * W_BYTES + w_off);
                w[i][0] = t2.x; w[i][V - 1] = t2.y;
            } else {
                const uint4 t4 = *reinterpret_cast<const uint4 *>(st + i * 32 * W_BYTES + w_off);
                w[i][0] = t4.x; w[i][1 % V] = t4.y; w[i][2 % V] = t4.z; w[i][3 % V] = t4.w;
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const uint2 t2 = *reinterpret_cast<const uint2 *>(st + x_off + mt * 32 * 8);
            xb[mt][0] = t2.x; xb[mt][1] = t2.y;
        }

#pragma unroll
        for (int mt = 0; mt < MT; mt++) mma_bf16_16816(sx[mt], ones, xb[mt]);

#pragma unroll
        for (int v = 0; v < V; v++) {
            // rows (4c, 4c+1) -> first k pair, rows (4c+2, 4c+3) -> second k pair
            const uint32_t pa[4] = {gather_byte<0>(w[0][v], w[1][v]), gather_byte<1>(w[0][v], w[1][v]),
                                    gather_byte<2>(w[0][v], w[1][v]), gather_byte<3>(w[0][v], w[1][v])};
            const uint32_t pb[4] = {gather_byte<0>(w[2][v], w[3][v]), gather_byte<1>(w[2][v], w[3][v]),
                                    gather_byte<2>(w[2][v], w[3][v]), gather_byte<3>(w[2][v], w[3][v])};
#pragma unroll
            for (int t = 0; t < 4; t++) {
                // tile t: MMA row g = column 2t of the word (slot t), row g+8 = column 2t+1 (slot t+4)
                uint32_t a[4];
                if (t & 1) {
                    a[0] = hi_nibbles_bf16(pa[t >> 1]); a[1] = hi_nibbles_bf16(pa[2 + (t >> 1)]);
                    a[2] = hi_nibbles_bf16(pb[t >> 1]); a[3] = hi_nibbles_bf16(pb[2 + (t >> 1)]);
                } else {
                    a[0] = lo_nibbles_bf16(pa[t >> 1]); a[1] = lo_nibbles_bf16(pa[2 + (t >> 1)]);
                    a[2] = lo_nibbles_bf16(pb[t >> 1]); a[3] = lo_nibbles_bf16(pb[2 + (t >> 1)]);
                }
#pragma unroll
                for (int mt = 0; mt < MT; mt++) mma_bf16_16816(acc[v][t][mt], a, xb[mt]);
            }
        }

        // End of a quantization group (or of this CTA's k range): fold scale and zero point in f32.
        const int k_next = (step_beg + s + 1) * 16;
        if ((k_next % p.group_size) == 0 || s == steps - 1) {
            const int grp = (k_next - 1) / p.group_size;
#pragma unroll
            for (int v = 0; v < V; v++) {
                const uint32_t zw = j_ok ? p.qzeros[(size_t)grp * p.packed_out + jbase + v] : 0u;
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const size_t n0 = (size_t)(jbase + v) * 8 + 2 * t;
                    const float s0 = j_ok ? load_as_f32(p.scales, p.scales_dtype, (size_t)grp * p.n + n0) : 0.0f;
                    const float s1 = j_ok ? load_as_f32(p.scales, p.scales_dtype, (size_t)grp * p.n + n0 + 1) : 0.0f;
                    const float z0 = 128.0f + (float)((zw >> (4 * t)) & 0xFu);
                    const float z1 = 128.0f + (float)((zw >> (4 * t + 16)) & 0xFu);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        float(&a4)[4] = acc[v][t][mt];
                        float(&t4)[4] = tot[v][t][mt];
                        t4[0] = fmaf(s0, fmaf(-z0, sx[mt][0], a4[0]), t4[0]);
                        t4[1] = fmaf(s0, fmaf(-z0, sx[mt][1], a4[1]), t4[1]);
                        t4[2] = fmaf(s1, fmaf(-z1, sx[mt][0], a4[2]), t4[2]);
                        t4[3] = fmaf(s1, fmaf(-z1, sx[mt][1], a4[3]), t4[3]);
                        a4[0] = a4[1] = a4[2] = a4[3] = 0.0f;
                    }
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) sx[mt][0] = sx[mt][1] = sx[mt][2] = sx[mt][3] = 0.0f;
        }
    }
    cp_async_wait<0>();

    // tot[v][t][mt][e]: token 8mt + 2c + (e&1), out column 8(jbase+v) + 2t + (e>>1)
    auto emit = [&](int v, int t, int mt, int e, float val) {
        const int row = 8 * mt + 2 * c + (e & 1);
        const size_t col = (size_t)(jbase + v) * 8 + 2 * t + (e >> 1);
        if (j_ok && row < p.m) {
            if (p.bias) val += load_as_f32(p.bias, p.bias_dtype, col);
            store_as(p.y, p.y_dtype, (size_t)row * p.n + col, val);
        }
    };

    if (nranks == 1) {
#pragma unroll
        for (int v = 0; v < V; v++)
#pragma unroll
            for (int t = 0; t < 4; t++)
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int e = 0; e < 4; e++) emit(v, t, mt, e, tot[v][t][mt][e]);
        return;
    }

    // Cluster reduction over the k split: every CTA publishes its partials in its
    // own shared memory, then CTA r sums accumulator slots a == r (mod nranks)
    // over the ranks in ascending order.
    cg::cluster_group cluster = cg::this_cluster();
    float *red = reinterpret_cast<float *>(smem);
    __syncthreads(); // every warp is done with its ring before it is reused
#pragma unroll
    for (int v = 0; v < V; v++)
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) red[(((v * 4 + t) * MT + mt) * 4 + e) * NT + tid] = tot[v][t][mt][e];
    cluster.sync();
#pragma unroll
    for (int v = 0; v < V; v++)
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int a = ((v * 4 + t) * MT + mt) * 4 + e;
                    if (a % nranks == rank) {
                        float sum = 0.0f;
                        for (int q = 0; q < nranks; q++) sum += cluster.map_shared_rank(red, q)[a * NT + tid];
                        emit(v, t, mt, e, sum);
                    }
                }
    cluster.sync(); // nobody leaves while a peer may still read its shared memory
    (void)NACC;
}


// ---------------------------------------------------------------------------
// Main variant: slices aligned to quantization groups, weights streamed straight
// into registers, f16 tensor cores.
//
// A CTA is KW warps on the SAME 8*V packed words (64*V out columns), each warp
// on its own contiguous k slice; a cluster of R such CTAs covers all of k.
// A slice is either a whole number of groups or a divisor of one group, so the
// scale/zero fold happens at most once per group into running f32 totals.
// Weights go from HBM to registers with streaming vector loads issued D steps
// ahead (plain loads sustain the stream; lane-private cp.async measured about
// half the rate). The CTA's slice of x is staged once in shared memory as f16
// (saturated to +-65504): with a 10-bit mantissa both nibbles of a byte become
// exact f16 values with one three-input lop3 and no shift -- 0x6400 | q is
// 1024 + q and 0x6400 | (q << 4) is 1024 + 16 q -- and the offsets and the
// factor 16 are taken out again in f32 when a group is folded. The integer pipe
// is the scarce resource here (one op per weight at half issue rate). Partials
// meet in (distributed) shared memory and every valid output is summed by one
// thread of the cluster in ascending k order.
constexpr int GK_KW = 4;

template <int V> __device__ __forceinline__ void ld_stream(uint32_t (&dst)[V], const uint32_t *p)
{
    if (V == 1) dst[0] = __ldcs(p);
    else if (V == 2) { const uint2 t = __ldcs(reinterpret_cast<const uint2 *>(p)); dst[0] = t.x; dst[V - 1] = t.y; }
    else { const uint4 t = __ldcs(reinterpret_cast<const uint4 *>(p)); dst[0] = t.x; dst[1 % V] = t.y; dst[2 % V] = t.z; dst[3 % V] = t.w; }
}

// (p & mask) | magic in one instruction (lut 0xEA = (a & b) | c). Mask and magic are passed in
// registers: a LOP3 encodes a single immediate, so with two literals the compiler re-materialises
// one of them with an extra move in front of every use.
__device__ __forceinline__ uint32_t and_or(uint32_t p, uint32_t mask, uint32_t magic)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(p), "r"(mask), "r"(magic));
    return r;
}

__device__ __forceinline__ void mma_f16_16816_awq(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int MT, int V, int D, int MINB>
__global__ void __launch_bounds__(GK_KW * 32, MINB) awq_gemv_group_kernel(const AwqGemvParams p)
{
    constexpr int KW = GK_KW;
    constexpr int NACC = V * 4 * MT * 4;
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();

    GV_CTA(0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, c = lane & 3;
    const int rank = blockIdx.y, nranks = gridDim.y;
    // Token tiles of one n tile sit in neighbouring CTAs: they stream the same weights at the same
    // time, so all but the first reader hit in L2.
    const int zt = blockIdx.x % p.token_split;
    const int m0 = zt * 8 * MT, m_loc = min(8 * MT, p.m - m0); // this CTA's tokens [m0, m0 + m_loc)
    const int jtile = (blockIdx.x / p.token_split) * 8 * V;
    const int jbase = jtile + g * V;
    const bool j_ok = jbase < p.packed_out;
    const int steps = p.steps_per_cta; // 16-row steps per warp slice, identical for all slices; a multiple of D
    const int gsteps = p.group_size >> 4;
    uint32_t mask_lo, mask_hi, kmagic; // opaque to constant propagation so that they stay in registers
    asm volatile("mov.b32 %0, 0x000F000F;\n\tmov.b32 %1, 0x00F000F0;\n\tmov.b32 %2, 0x64006400;"
                 : "=r"(mask_lo), "=r"(mask_hi), "=r"(kmagic));
    const int kr = KW * steps * 16;    // k range of this CTA
    const int k_cta = rank * kr;
    const int step_beg = (rank * KW + warp) * steps;

    // First weights on their way before anything else. Lanes past the last word re-read word 0
    // (their results are never stored).
    const size_t row_stride = (size_t)p.packed_out;
    const uint32_t *wsrc = p.qweight + (size_t)(step_beg * 16 + 4 * c) * row_stride + (j_ok ? jbase : 0);
    uint32_t buf[D][4][V];
#pragma unroll
    for (int d = 0; d < D; d++)
#pragma unroll
        for (int i = 0; i < 4; i++) ld_stream<V>(buf[d][i], wsrc + (size_t)(16 * d + i) * row_stride);

    // x[0 .. m) x [k_cta, k_cta + kr) -> shared memory as f16, rows padded by 32 bytes so that the
    // 8-byte fragment reads of a half warp (4 rows x 32 bytes) fall into distinct banks. Lanes whose
    // token does not exist read a block of zeros instead (stride 0).
    const int xrow = kr + 16; // elements
    __half *xs = reinterpret_cast<__half *>(smem);
    uint32_t *zeros = reinterpret_cast<uint32_t *>(smem + (size_t)m_loc * xrow * sizeof(__half));
    if (tid < 4) zeros[tid] = 0u;
    // Running totals live in shared memory, one 16-byte slot per (warp, MMA tile, lane), private to the
    // lane until the final reduction reads them: registers are kept for weights in flight instead.
    float4 *red = reinterpret_cast<float4 *>(zeros + 4);
    float4 *mine = red + (size_t)warp * (NACC / 4) * 32 + lane;
#pragma unroll
    for (int i = 0; i < NACC / 4; i++) mine[i * 32] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    pdl_wait(); // x may come from the kernel before this one; the first weights are already on their way
    for (int row = 0; row < m_loc; row++) {
        const uint2 *src = reinterpret_cast<const uint2 *>(p.x + (size_t)(m0 + row) * p.k + k_cta);
        uint2 *dst = reinterpret_cast<uint2 *>(xs + (size_t)row * xrow);
        for (int q4 = tid; q4 < (kr >> 2); q4 += KW * 32) {
            const uint2 raw = __ldg(src + q4);
            dst[q4] = make_uint2(f32x2_to_f16x2_sat(bf16_lo_f32(raw.x), bf16_hi_f32(raw.x)),
                                 f32x2_to_f16x2_sat(bf16_lo_f32(raw.y), bf16_hi_f32(raw.y)));
        }
    }

    // Zero points and scales of the slice's first group (16-bit scales ride in registers: reading them
    // only when the group is folded would stall the warp for a full memory round trip per group).
    const bool sc16 = p.scales_dtype != OXQ_F32;
    const bool is_f16 = p.scales_dtype == OXQ_F16;
    uint32_t zw[V], sraw[V][4];
    auto fetch_group = [&](int grp) {
#pragma unroll
        for (int v = 0; v < V; v++) {
            zw[v] = j_ok ? __ldg(p.qzeros + (size_t)grp * p.packed_out + jbase + v) : 0u;
            uint4 r = make_uint4(0u, 0u, 0u, 0u);
            if (j_ok && sc16)
                r = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.scales) +
                                                          (size_t)grp * p.n + (size_t)(jbase + v) * 8));
            sraw[v][0] = r.x; sraw[v][1] = r.y; sraw[v][2] = r.z; sraw[v][3] = r.w;
        }
    };
    int grp = (step_beg * 16) / p.group_size;
    fetch_group(grp);
    __syncthreads();
    GV_CTA(1);

    float acc[V][4][MT][4], sx[MT][4];
#pragma unroll
    for (int v = 0; v < V; v++)
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[v][t][mt][e] = 0.0f;
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) sx[mt][e] = 0.0f;

    // The group that just ended goes into the totals; acc and sum_x restart. Tile t holds columns
    // 2t and 2t+1 of the word (nibbles t and t+4). Even t used low nibbles, acc = sum (1024 + q) x:
    //   tot += s * acc - s * (1024 + z) * sum_x.
    // Odd t used high nibbles, acc = sum (1024 + 16 q) x:  tot += (s/16) * acc - s * (64 + z) * sum_x.
    auto fold = [&]() {
#pragma unroll
        for (int v = 0; v < V; v++) {
#pragma unroll
            for (int t = 0; t < 4; t++) {
                float s0, s1;
                if (sc16) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&sraw[v][t]));
                    const float b0 = __uint_as_float(sraw[v][t] << 16), b1 = __uint_as_float(sraw[v][t] & 0xFFFF0000u);
                    s0 = is_f16 ? f.x : b0;
                    s1 = is_f16 ? f.y : b1;
                } else {
                    const size_t n0 = (size_t)(jbase + v) * 8 + 2 * t;
                    s0 = j_ok ? reinterpret_cast<const float *>(p.scales)[(size_t)grp * p.n + n0] : 0.0f;
                    s1 = j_ok ? reinterpret_cast<const float *>(p.scales)[(size_t)grp * p.n + n0 + 1] : 0.0f;
                }
                const uint32_t zq = zw[v] >> (4 * t);
                const float off = (t & 1) ? 64.0f : 1024.0f;
                const float u0 = s0 * (off + (float)(zq & 0xFu)), u1 = s1 * (off + (float)((zq >> 16) & 0xFu));
                const float a0 = (t & 1) ? s0 * 0.0625f : s0, a1 = (t & 1) ? s1 * 0.0625f : s1;
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    float(&a4)[4] = acc[v][t][mt];
                    float4 &slot = mine[((v * 4 + t) * MT + mt) * 32];
                    float4 t4 = slot;
                    t4.x = fmaf(a0, a4[0], fmaf(-u0, sx[mt][0], t4.x));
                    t4.y = fmaf(a0, a4[1], fmaf(-u0, sx[mt][1], t4.y));
                    t4.z = fmaf(a1, a4[2], fmaf(-u1, sx[mt][0], t4.z));
                    t4.w = fmaf(a1, a4[3], fmaf(-u1, sx[mt][1], t4.w));
                    slot = t4;
                    a4[0] = a4[1] = a4[2] = a4[3] = 0.0f;
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++) sx[mt][0] = sx[mt][1] = sx[mt][2] = sx[mt][3] = 0.0f;
    };

    const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u}; // f16 1.0
    const __half *xw[MT];
    int xstep[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const bool real = 8 * mt + g < m_loc;
        xw[mt] = real ? xs + (size_t)(8 * mt + g) * xrow + warp * steps * 16 + 4 * c : reinterpret_cast<const __half *>(zeros);
        xstep[mt] = real ? 16 : 0;
    }
    int to_fold = min(steps, gsteps - (step_beg % gsteps)); // steps left in the current group

    for (int s0 = 0; s0 < steps; s0 += D) {
        const bool more = s0 + D < steps;
#pragma unroll
        for (int d = 0; d < D; d++) {
            uint32_t w[4][V], xb[MT][2];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int v = 0; v < V; v++) w[i][v] = buf[d][i][v];
            if (more) {
#pragma unroll
                for (int i = 0; i < 4; i++) ld_stream<V>(buf[d][i], wsrc + (size_t)(16 * (D + d) + i) * row_stride);
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const uint2 t2 = *reinterpret_cast<const uint2 *>(xw[mt]);
                xw[mt] += xstep[mt];
                xb[mt][0] = t2.x; xb[mt][1] = t2.y;
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) mma_f16_16816_awq(sx[mt], ones, xb[mt]);
#pragma unroll
            for (int v = 0; v < V; v++) {
                // rows (4c, 4c+1) -> first k pair, rows (4c+2, 4c+3) -> second k pair
                const uint32_t pa[4] = {gather_byte<0>(w[0][v], w[1][v]), gather_byte<1>(w[0][v], w[1][v]),
                                        gather_byte<2>(w[0][v], w[1][v]), gather_byte<3>(w[0][v], w[1][v])};
                const uint32_t pb[4] = {gather_byte<0>(w[2][v], w[3][v]), gather_byte<1>(w[2][v], w[3][v]),
                                        gather_byte<2>(w[2][v], w[3][v]), gather_byte<3>(w[2][v], w[3][v])};
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    // tile t: MMA row g = column 2t of the word (nibble t), row g+8 = column 2t+1 (nibble t+4)
                    const uint32_t mk = (t & 1) ? mask_hi : mask_lo;
                    const uint32_t a[4] = {and_or(pa[t >> 1], mk, kmagic), and_or(pa[2 + (t >> 1)], mk, kmagic),
                                           and_or(pb[t >> 1], mk, kmagic), and_or(pb[2 + (t >> 1)], mk, kmagic)};
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) mma_f16_16816_awq(acc[v][t][mt], a, xb[mt]);
                }
            }
            if (--to_fold == 0) {
                fold();
                const int done = s0 + d + 1;
                if (done < steps) {
                    grp += 1;
                    fetch_group(grp);
                    to_fold = min(gsteps, steps - done);
                }
            }
        }
        wsrc += (size_t)16 * D * row_stride;
    }
    GV_CTA(2);
    cg::cluster_group cluster = cg::this_cluster();
    if (nranks > 1) cluster.sync(); else __syncthreads();
    GV_CTA(3);

    // Every tile slot (tile, lane) that holds a real token is summed by one thread of the cluster
    // over the KW * R slices in ascending k order (bank-conflict-free: lane-minor, 16-byte loads).
    const int cluster_threads = nranks * KW * 32;
    for (int o = rank * KW * 32 + tid; o < (NACC / 4) * 32; o += cluster_threads) {
        const int tile = o >> 5, ol = o & 31;
        // tile = (v*4 + t)*MT + mt; components: token 8mt + 2c + {0,1}, out column 8(word) + 2t + {0,1}
        const int mt = tile % MT, vt = tile / MT, t = vt & 3, v = vt >> 2;
        const int og = ol >> 2, oc = ol & 3;
        const int word = jtile + og * V + v;
        const int row = 8 * mt + 2 * oc;
        if (word < p.packed_out && row < m_loc) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int q = 0; q < nranks; q++) {
                const float4 *src = nranks > 1 ? cluster.map_shared_rank(red, q) : red;
#pragma unroll
                for (int ks = 0; ks < KW; ks++) {
                    const float4 pv = src[((size_t)ks * (NACC / 4) + tile) * 32 + ol];
                    sum.x += pv.x; sum.y += pv.y; sum.z += pv.z; sum.w += pv.w;
                }
            }
            const size_t col = (size_t)word * 8 + 2 * t;
            float b0 = 0.0f, b1 = 0.0f;
            if (p.bias) { b0 = load_as_f32(p.bias, p.bias_dtype, col); b1 = load_as_f32(p.bias, p.bias_dtype, col + 1); }
            store_as(p.y, p.y_dtype, (size_t)(m0 + row) * p.n + col, sum.x + b0);
            store_as(p.y, p.y_dtype, (size_t)(m0 + row) * p.n + col + 1, sum.z + b1);
            if (row + 1 < m_loc) {
                store_as(p.y, p.y_dtype, (size_t)(m0 + row + 1) * p.n + col, sum.y + b0);
                store_as(p.y, p.y_dtype, (size_t)(m0 + row + 1) * p.n + col + 1, sum.w + b1);
            }
        }
    }
    GV_CTA(4);
    if (nranks > 1) cluster.sync();
    GV_CTA(5);
}

template <int MT, int V, int D, int MINB>
static int launch_awq_gemv_group(const AwqGemvParams &p, int nranks, cudaStream_t stream)
{
    constexpr int NACC = V * 4 * MT * 4;
    const int m_cta = p.m < 8 * MT ? p.m : 8 * MT;
    const size_t xbytes = (size_t)m_cta * (GK_KW * p.steps_per_cta * 16 + 16) * sizeof(__half) + 16;
    const size_t red = (size_t)GK_KW * NACC * 32 * sizeof(float);
    const size_t smem = xbytes + red;
    auto kern = awq_gemv_group_kernel<MT, V, D, MINB>;
    static size_t configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || configured[device] < smem) {
        OXQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (device < 64) configured[device] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ceil_div(p.packed_out, 8 * V) * p.token_split, nranks, 1);
    cfg.blockDim = dim3(GK_KW * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = nranks;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    allow_early_start(attr, cfg.numAttrs);
    OXQ_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return OXQ_OK;
}

// ---------------------------------------------------------------------------
// TMA-ring variant of the main kernel (same slicing, same arithmetic, same fixed-order reduction).
//
// The register-streaming kernel above keeps at most D steps of weights in flight per warp, because
// bytes in flight are registers; at four CTAs per SM that is about 25 KB per SM, well short of what
// the memory system needs to stay busy. Here every warp owns a ring of `stages` shared-memory slots;
// lane 0 asks the TMA unit for one box of GT_ROWS input rows x 16 packed words (2 KB) per slot and
// refills a slot as soon as the warp has read it, so a warp keeps stages x 2 KB on their way with one
// instruction per box and no registers. A box lands as dense 64-byte rows. Within a 16-row step lane
// (g, c) reads rows c, 4 + c, 8 + c, 12 + c (consecutive rows across c: the four rows of one
// instruction are 256 contiguous bytes); x is staged in the matching order, so element 4c + i of a
// 16-block is x[4i + c] and a lane's B fragment is still one 8-byte read.
constexpr int GT_KW = 4;
constexpr int GT_ROWS = 32;
constexpr int GT_STAGE_BYTES = GT_ROWS * 64;
constexpr int GT_MAX_STAGES = 8;

__device__ int g_awq_gemv_flag; // non-zero after a wait on a weight box gave up

template <int MT, int MINB>
__global__ void __launch_bounds__(GT_KW * 32, MINB)
    awq_gemv_tma_kernel(const AwqGemvParams p, const __grid_constant__ CUtensorMap wmap)
{
    constexpr int KW = GT_KW, V = 2;
    constexpr int NACC = V * 4 * MT * 4;
    extern __shared__ __align__(1024) unsigned char smem_ring[]; // TMA destinations want 128-byte alignment

    GV_CTA(0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, c = lane & 3;
    const int rank = blockIdx.y, nranks = gridDim.y;
    const int zt = blockIdx.x % p.token_split;
    const int m0 = zt * 8 * MT, m_loc = min(8 * MT, p.m - m0);
    const int jtile = (blockIdx.x / p.token_split) * 8 * V;
    const int jbase = jtile + g * V;
    const int steps = p.steps_per_cta; // 16-row steps per warp slice (even)
    const int boxes = steps >> 1;
    const int gsteps = p.group_size >> 4;
    const int S = p.stages;
    uint32_t mask_lo, mask_hi, kmagic;
    asm volatile("mov.b32 %0, 0x000F000F;\n\tmov.b32 %1, 0x00F000F0;\n\tmov.b32 %2, 0x64006400;"
                 : "=r"(mask_lo), "=r"(mask_hi), "=r"(kmagic));
    const int kr = KW * steps * 16;
    const int k_cta = rank * kr;
    const int step_beg = (rank * KW + warp) * steps;

    // shared memory: rings | barriers | x | zeros | totals
    unsigned char *ring = smem_ring + (size_t)warp * S * GT_STAGE_BYTES;
    const uint32_t ring_addr = smem_u32(ring);
    const uint32_t bar0 = smem_u32(smem_ring + (size_t)KW * S * GT_STAGE_BYTES) + warp * GT_MAX_STAGES * 8;
    unsigned char *rest = smem_ring + (size_t)KW * S * GT_STAGE_BYTES + KW * GT_MAX_STAGES * 8;

    // The next launch on the stream may start its own weight boxes while this one drains; nothing
    // that another kernel may have produced (x) or may still read (y) is touched before the wait below.
    pdl_launch_dependents();
    if (nranks > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); // met again before the first remote store

    if (lane == 0) {
        for (int s = 0; s < S; s++) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int s = 0; s < S && s < boxes; s++) {
            mbar_arrive_expect_tx(bar0 + 8 * s, GT_STAGE_BYTES);
            tma_load_2d(ring_addr + s * GT_STAGE_BYTES, &wmap, bar0 + 8 * s, jtile, step_beg * 16 + s * GT_ROWS);
        }
    }
    __syncwarp();

    const int xrow = kr + 16; // elements; the 32-byte pad keeps the fragment reads of four tokens in distinct banks
    __half *xs = reinterpret_cast<__half *>(rest);
    uint32_t *zeros = reinterpret_cast<uint32_t *>(rest + (size_t)m_loc * xrow * sizeof(__half));
    if (tid < 4) zeros[tid] = 0u;
    float4 *red = reinterpret_cast<float4 *>(zeros + 4);
    float4 *mine = red + (size_t)warp * (NACC / 4) * 32 + lane;
    float4 *inbox = red + (size_t)KW * (NACC / 4) * 32; // [source rank][local tile][lane], written by the whole cluster
#pragma unroll
    for (int i = 0; i < NACC / 4; i++) mine[i * 32] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);

    const bool sc16 = p.scales_dtype != OXQ_F32;
    const bool is_f16 = p.scales_dtype == OXQ_F16;
    uint32_t zw[V], sraw[V][4];
    auto fetch_group = [&](int grp) {
#pragma unroll
        for (int v = 0; v < V; v++) {
            zw[v] = __ldg(p.qzeros + (size_t)grp * p.packed_out + jbase + v);
            uint4 r = make_uint4(0u, 0u, 0u, 0u);
            if (sc16)
                r = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.scales) +
                                                          (size_t)grp * p.n + (size_t)(jbase + v) * 8));
            sraw[v][0] = r.x; sraw[v][1] = r.y; sraw[v][2] = r.z; sraw[v][3] = r.w;
        }
    };
    int grp = (step_beg * 16) / p.group_size;
    fetch_group(grp);

    pdl_wait();
    {   // x[m0 .. m0 + m_loc) x [k_cta, k_cta + kr) -> f16 in the order the fragments want; loads of four items
        // are issued before the first is converted, so the staging costs about one memory round trip.
        const int per = kr >> 2, items = m_loc * per;
        for (int base = tid; base < items; base += 4 * KW * 32) {
            uint2 raw[4];
            int at[4];
#pragma unroll
            for (int j4 = 0; j4 < 4; j4++) {
                const int idx = base + j4 * KW * 32;
                at[j4] = -1;
                if (idx < items) {
                    const int row = idx / per, q4 = idx - row * per;
                    raw[j4] = __ldg(reinterpret_cast<const uint2 *>(p.x + (size_t)(m0 + row) * p.k + k_cta) + q4);
                    at[j4] = row * xrow + (q4 >> 2) * 16 + (q4 & 3); // x[16 blk + 4 i + cc] -> element 16 blk + 4 cc + i
                }
            }
#pragma unroll
            for (int j4 = 0; j4 < 4; j4++) {
                if (at[j4] < 0) continue;
                const uint32_t h01 = f32x2_to_f16x2_sat(bf16_lo_f32(raw[j4].x), bf16_hi_f32(raw[j4].x));
                const uint32_t h23 = f32x2_to_f16x2_sat(bf16_lo_f32(raw[j4].y), bf16_hi_f32(raw[j4].y));
                unsigned short *d16 = reinterpret_cast<unsigned short *>(xs) + at[j4];
                d16[0] = (unsigned short)(h01 & 0xFFFFu);
                d16[4] = (unsigned short)(h01 >> 16);
                d16[8] = (unsigned short)(h23 & 0xFFFFu);
                d16[12] = (unsigned short)(h23 >> 16);
            }
        }
    }
    __syncthreads();
    GV_CTA(1);

    float acc[V][4][MT][4], sx[MT][4];
#pragma unroll
    for (int v = 0; v < V; v++)
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[v][t][mt][e] = 0.0f;
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) sx[mt][e] = 0.0f;

    // Same fold as the register-streaming kernel: even tiles carry 1024 + q, odd tiles 1024 + 16 q.
    auto fold = [&]() {
#pragma unroll
        for (int v = 0; v < V; v++) {
#pragma unroll
            for (int t = 0; t < 4; t++) {
                float s0, s1;
                if (sc16) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&sraw[v][t]));
                    const float b0 = __uint_as_float(sraw[v][t] << 16), b1 = __uint_as_float(sraw[v][t] & 0xFFFF0000u);
                    s0 = is_f16 ? f.x : b0;
                    s1 = is_f16 ? f.y : b1;
                } else {
                    const size_t n0 = (size_t)(jbase + v) * 8 + 2 * t;
                    s0 = reinterpret_cast<const float *>(p.scales)[(size_t)grp * p.n + n0];
                    s1 = reinterpret_cast<const float *>(p.scales)[(size_t)grp * p.n + n0 + 1];
                }
                const uint32_t zq = zw[v] >> (4 * t);
                const float off = (t & 1) ? 64.0f : 1024.0f;
                const float u0 = s0 * (off + (float)(zq & 0xFu)), u1 = s1 * (off + (float)((zq >> 16) & 0xFu));
                const float a0 = (t & 1) ? s0 * 0.0625f : s0, a1 = (t & 1) ? s1 * 0.0625f : s1;
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    float(&a4)[4] = acc[v][t][mt];
                    float4 &slot = mine[((v * 4 + t) * MT + mt) * 32];
                    float4 t4 = slot;
                    t4.x = fmaf(a0, a4[0], fmaf(-u0, sx[mt][0], t4.x));
                    t4.y = fmaf(a0, a4[1], fmaf(-u0, sx[mt][1], t4.y));
                    t4.z = fmaf(a1, a4[2], fmaf(-u1, sx[mt][0], t4.z));
                    t4.w = fmaf(a1, a4[3], fmaf(-u1, sx[mt][1], t4.w));
                    slot = t4;
                    a4[0] = a4[1] = a4[2] = a4[3] = 0.0f;
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++) sx[mt][0] = sx[mt][1] = sx[mt][2] = sx[mt][3] = 0.0f;
    };

    const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u}; // f16 1.0
    const __half *xw[MT];
    int xstep[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const bool real = 8 * mt + g < m_loc;
        xw[mt] = real ? xs + (size_t)(8 * mt + g) * xrow + warp * steps * 16 + 4 * c : reinterpret_cast<const __half *>(zeros);
        xstep[mt] = real ? 16 : 0;
    }
    int to_fold = min(steps, gsteps - (step_beg % gsteps));
    const uint32_t lane_off = (uint32_t)c * 64 + g * 8;

    int slot = 0, phase = 0, done = 0;
    for (int it = 0; it < boxes; it++) {
        if (!mbar_wait(bar0 + 8 * slot, phase, &g_awq_gemv_flag, 1)) break;
        const unsigned char *st = ring + (size_t)slot * GT_STAGE_BYTES + lane_off;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t w[4][V], xb[MT][2];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint2 t2 = *reinterpret_cast<const uint2 *>(st + (h * 16 + 4 * i) * 64);
                w[i][0] = t2.x; w[i][1] = t2.y;
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const uint2 t2 = *reinterpret_cast<const uint2 *>(xw[mt]);
                xw[mt] += xstep[mt];
                xb[mt][0] = t2.x; xb[mt][1] = t2.y;
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) mma_f16_16816_awq(sx[mt], ones, xb[mt]);
#pragma unroll
            for (int v = 0; v < V; v++) {
                const uint32_t pa[4] = {gather_byte<0>(w[0][v], w[1][v]), gather_byte<1>(w[0][v], w[1][v]),
                                        gather_byte<2>(w[0][v], w[1][v]), gather_byte<3>(w[0][v], w[1][v])};
                const uint32_t pb[4] = {gather_byte<0>(w[2][v], w[3][v]), gather_byte<1>(w[2][v], w[3][v]),
                                        gather_byte<2>(w[2][v], w[3][v]), gather_byte<3>(w[2][v], w[3][v])};
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const uint32_t mk = (t & 1) ? mask_hi : mask_lo;
                    const uint32_t a[4] = {and_or(pa[t >> 1], mk, kmagic), and_or(pa[2 + (t >> 1)], mk, kmagic),
                                           and_or(pb[t >> 1], mk, kmagic), and_or(pb[2 + (t >> 1)], mk, kmagic)};
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) mma_f16_16816_awq(acc[v][t][mt], a, xb[mt]);
                }
            }
            done += 1;
            if (--to_fold == 0) {
                fold();
                if (done < steps) {
                    grp += 1;
                    fetch_group(grp);
                    to_fold = min(gsteps, steps - done);
                }
            }
        }
        __syncwarp(); // every lane has read the slot
        if (lane == 0 && it + S < boxes) {
            mbar_arrive_expect_tx(bar0 + 8 * slot, GT_STAGE_BYTES);
            tma_load_2d(ring_addr + slot * GT_STAGE_BYTES, &wmap, bar0 + 8 * slot, jtile, step_beg * 16 + (it + S) * GT_ROWS);
        }
        if (++slot == S) { slot = 0; phase ^= 1; }
    }
    GV_CTA(2);
    // Reduction: every CTA adds its KW warp slices (ascending k) and sends the sum of tile t to the CTA
    // that owns it (t % nranks); after one cluster barrier the owner adds the nranks partial sums in
    // rank order (ascending k again) and stores. Nobody reads another CTA's memory, so a CTA may leave
    // right after the barrier.
    constexpr int NT = NACC / 4;
    const int LT = (NT + nranks - 1) / nranks;
    cg::cluster_group cluster = cg::this_cluster();
    __syncthreads();
    if (nranks > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); // every CTA of the cluster has started
    for (int o = tid; o < NT * 32; o += KW * 32) {
        const int tile = o >> 5, ol = o & 31;
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int ks = 0; ks < KW; ks++) {
            const float4 pv = red[((size_t)ks * NT + tile) * 32 + ol];
            sum.x += pv.x; sum.y += pv.y; sum.z += pv.z; sum.w += pv.w;
        }
        const int owner = tile % nranks, lt = tile / nranks;
        float4 *dst = nranks > 1 ? cluster.map_shared_rank(inbox, owner) : inbox;
        dst[((size_t)rank * LT + lt) * 32 + ol] = sum;
    }
    if (nranks > 1) cluster.sync(); else __syncthreads();
    GV_CTA(3);
    for (int o = tid; o < LT * 32; o += KW * 32) {
        const int lt = o >> 5, ol = o & 31;
        const int tile = lt * nranks + rank;
        if (tile >= NT) continue;
        const int mt = tile % MT, vt = tile / MT, t = vt & 3, v = vt >> 2;
        const int og = ol >> 2, oc = ol & 3;
        const int word = jtile + og * V + v;
        const int row = 8 * mt + 2 * oc;
        if (row < m_loc) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int q = 0; q < nranks; q++) {
                const float4 pv = inbox[((size_t)q * LT + lt) * 32 + ol];
                sum.x += pv.x; sum.y += pv.y; sum.z += pv.z; sum.w += pv.w;
            }
            const size_t col = (size_t)word * 8 + 2 * t;
            float b0 = 0.0f, b1 = 0.0f;
            if (p.bias) { b0 = load_as_f32(p.bias, p.bias_dtype, col); b1 = load_as_f32(p.bias, p.bias_dtype, col + 1); }
            store_as(p.y, p.y_dtype, (size_t)(m0 + row) * p.n + col, sum.x + b0);
            store_as(p.y, p.y_dtype, (size_t)(m0 + row) * p.n + col + 1, sum.z + b1);
            if (row + 1 < m_loc) {
                store_as(p.y, p.y_dtype, (size_t)(m0 + row + 1) * p.n + col, sum.y + b0);
                store_as(p.y, p.y_dtype, (size_t)(m0 + row + 1) * p.n + col + 1, sum.w + b1);
            }
        }
    }
    GV_CTA(4);
    GV_CTA(5);
}

template <int MT, int MINB>
static int launch_awq_gemv_tma(AwqGemvParams p, int nranks, cudaStream_t stream)
{
    constexpr int NACC = 2 * 4 * MT * 4;
    CUtensorMap wmap;
    const CUresult r = encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, p.qweight, (uint64_t)p.packed_out, (uint64_t)p.k,
                                       (uint64_t)p.packed_out * 4, 16, GT_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    OXQ_REQUIRE(r == CUDA_SUCCESS, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);

    const int m_cta = p.m < 8 * MT ? p.m : 8 * MT;
    const size_t xbytes = (size_t)m_cta * (GT_KW * p.steps_per_cta * 16 + 16) * sizeof(__half) + 16;
    const size_t inbox = (size_t)nranks * ceil_div(NACC / 4, nranks) * 32 * sizeof(float4);
    const size_t red = (size_t)GT_KW * NACC * 32 * sizeof(float) + inbox;
    const size_t fixed = xbytes + red + GT_KW * GT_MAX_STAGES * 8;
    // As many ring slots as still let MINB CTAs share an SM (228 KB, 1 KB reserved per CTA), at most the boxes of a slice.
    const size_t per_cta = (size_t)(228 * 1024) / MINB - 1024;
    int stages = per_cta > fixed ? (int)((per_cta - fixed) / (GT_KW * GT_STAGE_BYTES)) : 0;
    if (stages > GT_MAX_STAGES) stages = GT_MAX_STAGES;
    if (stages > p.steps_per_cta / 2) stages = p.steps_per_cta / 2;
    if (const char *env = tuning_env("OXQ_AWQ_GEMV_STAGES")) stages = atoi(env) < stages ? atoi(env) : stages;
    if (stages < 2) return OXQ_ERR_UNSUPPORTED; // the caller falls back to the register-streaming kernel
    p.stages = stages;
    const size_t smem = (size_t)GT_KW * stages * GT_STAGE_BYTES + fixed;

    auto kern = awq_gemv_tma_kernel<MT, MINB>;
    static size_t configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || configured[device] < smem) {
        OXQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (device < 64) configured[device] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.packed_out / 16) * p.token_split, nranks, 1);
    cfg.blockDim = dim3(GT_KW * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = nranks;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    allow_early_start(attr, cfg.numAttrs);
    OXQ_CUDA(cudaLaunchKernelEx(&cfg, kern, p, wmap));
    return OXQ_OK;
}

template <int MT, int V, int NW>
static int launch_awq_gemv(const AwqGemvParams &p, int ksplit, cudaStream_t stream)
{
    constexpr int NACC = V * 4 * MT * 4;
    constexpr int STAGE_BYTES = 32 * (16 * V + 8 * MT);
    const size_t ring = (size_t)NW * GEMV_STAGES * STAGE_BYTES;
    const size_t red = (size_t)NACC * NW * 32 * sizeof(float);
    const size_t smem = ring > red ? ring : red;
    auto kern = awq_gemv_kernel<MT, V, NW>;
    // Per-device, once: the attribute call is not a stream operation and must stay out of graph captures.
    static bool configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device < 64 && !configured[device]) {
        OXQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[device] = true;
    } else if (device >= 64) {
        OXQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ceil_div(p.packed_out, 8 * V * NW), ksplit, 1);
    cfg.blockDim = dim3(NW * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ksplit;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    OXQ_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return OXQ_OK;
}

} // namespace oxq

using namespace oxq;

OXQ_EXPORT int oxq_awq_gemv(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                            const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y,
                            int y_dtype, int m, int k, int n, int group_size, void *stream)
{
    clear_error();
    OXQ_REQUIRE(x && qweight && qzeros && scales && y, OXQ_ERR_NULL, "oxq_awq_gemv: null pointer");
    OXQ_REQUIRE(x_dtype == OXQ_BF16, OXQ_ERR_UNSUPPORTED, "oxq_awq_gemv: activations must be bf16");
    OXQ_REQUIRE(valid_dtype(scales_dtype) && valid_dtype(y_dtype) && (!bias || valid_dtype(bias_dtype)),
                OXQ_ERR_UNSUPPORTED, "oxq_awq_gemv: unsupported dtype");
    OXQ_REQUIRE(m >= 1 && m <= 32, OXQ_ERR_BAD_SHAPE, "oxq_awq_gemv: m=%d outside 1..32 (use the GEMM entry)", m);
    OXQ_REQUIRE(k > 0 && n > 0 && group_size > 0, OXQ_ERR_BAD_SHAPE, "oxq_awq_gemv: non-positive size");
    OXQ_REQUIRE(n % 8 == 0, OXQ_ERR_BAD_SHAPE, "AWQ out_features (%d) not divisible by pack factor 8", n);
    OXQ_REQUIRE(k % group_size == 0, OXQ_ERR_BAD_SHAPE, "quant in_features (%d) not divisible by group size (%d)", k,
                group_size);
    OXQ_REQUIRE((group_size & (group_size - 1)) == 0, OXQ_ERR_BAD_SHAPE, "group_size %d is not a power of two",
                group_size);
    OXQ_REQUIRE(group_size % 16 == 0 && k % 16 == 0, OXQ_ERR_UNSUPPORTED,
                "oxq_awq_gemv: group_size (%d) and in_features (%d) must be multiples of 16", group_size, k);
    OXQ_REQUIRE(aligned(x, 16) && aligned(qweight, 16) && aligned(qzeros, 4) && aligned(scales, 4) && aligned(y, 4),
                OXQ_ERR_BAD_ALIGN, "oxq_awq_gemv: x/qweight must be 16-byte aligned");

    AwqGemvParams p;
    p.x = (const __nv_bfloat16 *)x;
    p.qweight = qweight; p.qzeros = qzeros; p.scales = scales; p.bias = bias; p.y = y;
    p.scales_dtype = scales_dtype; p.bias_dtype = bias_dtype; p.y_dtype = y_dtype;
    p.m = m; p.k = k; p.n = n; p.group_size = group_size;
    p.packed_out = n / 8;

    const int mt = m <= 8 ? 1 : (m <= 16 ? 2 : 4);
    int v = mt == 4 ? 1 : 2;
    if (p.packed_out % v != 0) v = 1;
    constexpr int NW = 4;
    const int total_steps = k / 16;
    cudaStream_t st = (cudaStream_t)stream;

    // Main path: contiguous k slices, 4 warps x R CTAs, each slice a whole number of groups or a
    // divisor of one group. A CTA takes 8 * mtc tokens; more tokens go to neighbouring CTAs of the
    // same n tile (token split).
    p.token_split = 1;
    {
        // Measured on K = 4096, N = 14336: up to 8 tokens one CTA column with k split in 4; 9..16 tokens
        // 16 tokens per CTA, k split in 2; more tokens 8 per CTA on neighbouring CTAs, k split in 2.
        int fv = 2, mtc = (m > 8 && m <= 16) ? 2 : 1, r_force = 0, depth = 2, minb = 4;
        bool ok = aligned(scales, 16);
        if (const char *env = tuning_env("OXQ_AWQ_GEMV_FAST")) { // bench-harness knob: "0" disables, else "V[,R[,D[,B[,MT]]]]"
            int ev = 0, er = 0, ed = 0, eb = 0, em = 0;
            const int got = sscanf(env, "%d,%d,%d,%d,%d", &ev, &er, &ed, &eb, &em);
            if (got >= 1 && ev == 0) ok = false;
            if (got >= 1 && (ev == 1 || ev == 2 || ev == 4)) fv = ev;
            if (got >= 2 && (er == 1 || er == 2 || er == 4 || er == 8)) r_force = er;
            if (got >= 3 && (ed == 2 || ed == 4)) depth = ed;
            if (got >= 4 && eb == 6) minb = 6;
            if (got >= 5 && (em == 1 || em == 2 || em == 4)) mtc = em;
        }
        while (fv > 1 && p.packed_out % fv != 0) fv /= 2;
        const int split = ceil_div(m, 8 * mtc);
        const int m_cta = m < 8 * mtc ? m : 8 * mtc;
        const int gsteps = group_size / 16;
        const int n_tiles = ceil_div(p.packed_out, 8 * fv) * split;
        int r = 0;
        for (int cand : {8, 4, 2, 1}) {
            if (total_steps % (GK_KW * cand) != 0) continue;
            const int sl = total_steps / (GK_KW * cand);
            if (!(sl % gsteps == 0 || gsteps % sl == 0) || sl % depth != 0) continue;
            if ((size_t)m_cta * (GK_KW * sl * 16 + 16) * 2 > 160 * 1024) continue;
            if (r_force ? cand == r_force : (r == 0 || (m > 8 ? cand >= 2 : n_tiles * GK_KW * cand >= 1700))) r = cand;
        }
        if (ok && r != 0) {
            p.steps_per_cta = total_steps / (GK_KW * r);
            p.token_split = split;
            // TMA ring when the shape tiles into 16-word boxes and two-step slots.
            const char *tma_env = tuning_env("OXQ_AWQ_GEMV_TMA");
            if (fv == 2 && p.packed_out % 16 == 0 && p.steps_per_cta % 2 == 0 && !(tma_env && tma_env[0] == '0')) {
                // (a 16-token variant of the same kernel needs 156 registers and 80 KB per CTA: two waves, slower)
                const int rc = mtc == 1 ? launch_awq_gemv_tma<1, 4>(p, r, st) : OXQ_ERR_UNSUPPORTED;
                if (rc != OXQ_ERR_UNSUPPORTED) return rc;
            }
            if (mtc == 1 && fv == 4) return launch_awq_gemv_group<1, 4, 2, 2>(p, r, st);
            if (mtc == 1 && fv == 2 && depth == 2 && minb == 6) return launch_awq_gemv_group<1, 2, 2, 6>(p, r, st);
            if (mtc == 1 && fv == 2 && depth == 2) return launch_awq_gemv_group<1, 2, 2, 4>(p, r, st);
            if (mtc == 1 && fv == 2) return launch_awq_gemv_group<1, 2, 4, 4>(p, r, st);
            if (mtc == 1 && fv == 1) return launch_awq_gemv_group<1, 1, 4, 4>(p, r, st);
            if (mtc == 2 && fv == 2) return launch_awq_gemv_group<2, 2, 2, 2>(p, r, st);
            if (mtc == 2 && fv == 1) return launch_awq_gemv_group<2, 1, 2, 4>(p, r, st);
            if (mtc == 4 && fv == 1) return launch_awq_gemv_group<4, 1, 2, 2>(p, r, st);
            p.token_split = 1;
        }
    }

    // Enough CTAs for about two per SM; the k split is the cluster size (portable maximum 8).
    const int n_tiles = ceil_div(p.packed_out, 8 * v * NW);
    int ksplit = 1;
    while (ksplit < 8 && n_tiles * ksplit < 2 * sm_count() && total_steps / (ksplit * 2) >= 4) ksplit *= 2;
    if (const char *env = tuning_env("OXQ_AWQ_GEMV_TUNE")) { // bench-harness knob: "V,KSPLIT"
        int ev = 0, ek = 0;
        if (sscanf(env, "%d,%d", &ev, &ek) == 2) {
            if ((ev == 1 || ev == 2 || ev == 4) && p.packed_out % ev == 0 && 16 * ev * mt <= 64) v = ev;
            if (ek == 1 || ek == 2 || ek == 4 || ek == 8) ksplit = ek;
        }
    }
    p.steps_per_cta = ceil_div(total_steps, ksplit);
    if (mt == 1 && v == 1) return launch_awq_gemv<1, 1, NW>(p, ksplit, st);
    if (mt == 1 && v == 2) return launch_awq_gemv<1, 2, NW>(p, ksplit, st);
    if (mt == 1 && v == 4) return launch_awq_gemv<1, 4, NW>(p, ksplit, st);
    if (mt == 2 && v == 1) return launch_awq_gemv<2, 1, NW>(p, ksplit, st);
    if (mt == 2 && v == 2) return launch_awq_gemv<2, 2, NW>(p, ksplit, st);
    return launch_awq_gemv<4, 1, NW>(p, ksplit, st);
}

OXQ_EXPORT int oxq_awq_gemv_check(void *stream)
{
    clear_error();
    OXQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    int flag = 0;
    OXQ_CUDA(cudaMemcpyFromSymbol(&flag, g_awq_gemv_flag, sizeof(int)));
    if (flag != 0) { // report once
        const int zero = 0;
        OXQ_CUDA(cudaMemcpyToSymbol(g_awq_gemv_flag, &zero, sizeof(int)));
    }
    OXQ_REQUIRE(flag == 0, OXQ_ERR_DEVICE_FLAG,
                "oxq_awq_gemv: a bounded wait on a weight box ran out in a call since the last check (outputs of those calls are not valid)");
    return OXQ_OK;
}

#ifdef OXQ_TUNING
OXQ_EXPORT int oxq_gv_cta_read(unsigned long long *host_out)
{
    return cudaMemcpyFromSymbol(host_out, g_gv_cta, sizeof(unsigned long long) * 1024 * 8) == cudaSuccess ? 0 : -6;
}
#endif
