// C-ABI entry points of the prefill-sized (m > 32) quantized matmuls: dequantize a slab of weight
// rows into the caller's workspace (bit-exact kernels of dequant.cu), run the tcgen05 GEMM of
// gemm_tc.cu on it, repeat. A weight of up to 128 MiB (as bf16) is one slab; larger ones are cut so that each slab is a
// whole number of rounds of the persistent GEMM grid.
#include "oxq_common.cuh"

namespace oxq {
int gemm_bf16_tn(const void *x, const void *w, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int n,
                 int k, int n_off, int ldy, int *flag, cudaStream_t stream, int epi = 0);
int awq_dequant_rows_bf16(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                          __nv_bfloat16 *out, int k, int n_full, int group_size, int n_off, int n_cnt, cudaStream_t st,
                          int row_mul = 1, int row_add = 0);
int gptq_dequant_rows_bf16(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                           __nv_bfloat16 *out, int k, int n_full, int group_size, int bits, int sym, int n_off,
                           int n_cnt, cudaStream_t st);
int w8a16_dequant_rows_bf16(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                            __nv_bfloat16 *out, int k, int n_full, int group_size, int n_off, int n_cnt, cudaStream_t st);
int gguf_dequant_rows_bf16(int ggml_type, const uint8_t *blocks, __nv_bfloat16 *out, int k, int n_off, int n_cnt,
                           cudaStream_t st);
int fp8_dequant_rows_bf16(const uint8_t *weight, const float *scale_inv, int s_in, int block_out, int block_in,
                          __nv_bfloat16 *out, int k, int n_off, int n_cnt, cudaStream_t st);
int mxfp4_dequant_rows_bf16(const uint8_t *blocks, const uint8_t *scales, __nv_bfloat16 *out, int k, int n_off,
                            int n_cnt, cudaStream_t st);
bool gguf_block_layout_host(int ggml_type, int &bel, int &bby);
bool awq_fused_supported(int m, int k, int n, int group_size, int scales_dtype, const void *x, const void *qweight,
                         const void *scales);
bool fp8_fused_supported(int m, int k, int n, int block_out, int block_in, const void *x, const void *weight, const void *scale_inv);
int fp8_fused_matmul(const void *x, const uint8_t *weight, const float *scale_inv, int s_in, int block_out, int block_in,
                     const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n, int *flag, cudaStream_t st,
                     void *scratch, size_t scratch_bytes);
int awq_fused_matmul(const void *x, const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype, const void *bias,
                     int bias_dtype, void *y, int y_dtype, int m, int k, int n, int group_size, int col_base, int ldy,
                     int *flag, cudaStream_t st, int gptq, int sym, void *scratch, size_t scratch_bytes);

constexpr size_t WS_HEADER = 256;                // flag word + padding, keeps the slab 256-byte aligned
constexpr size_t SLAB_LIMIT_BYTES = 128u << 20;  // dequantized rows held at once (whole weight if it fits)

// Rows of the workspace slab for an [n, k] weight: everything if it fits the limit, else the limit.
static int slab_rows(int n, int k)
{
    long long rows = (long long)(SLAB_LIMIT_BYTES / ((size_t)k * 2)) / 256 * 256;
    if (rows < 256) rows = 256;
    return rows >= n ? n : (int)rows;
}

// When the weight needs several slabs, make each one a whole number of persistent-grid rounds:
// tiles_m x (rows / 256) tiles should be a multiple of the SM count.
static int slab_rows_for_m(int cap_rows, int n, int m)
{
    if (cap_rows >= n) return n;
    const int tiles_m = (m + 127) / 128;
    const int sms = sm_count();
    int g = tiles_m, b = sms;
    while (b) { const int t = g % b; g = b; b = t; } // gcd(tiles_m, SM count)
    const int q = sms / g * 256;                      // rows per balanced group of n tiles
    if (q <= cap_rows) return cap_rows / q * q;
    return cap_rows / 256 * 256;
}

struct GemmCommon {
    const void *x, *bias;
    void *y;
    int bias_dtype, y_dtype, m, k, n;
    int *flag;
    __nv_bfloat16 *slab;
    size_t slab_bytes = 0; // what the workspace holds behind the header
    int rows;
    cudaStream_t st;
    // tensor-parallel placement (oxq_awq_gemm_tp): this call's weight is columns [col_base, col_base + n) of an
    // output with `ldy` columns
    int col_base = 0, ldy = 0;
};

static int prepare(const char *who, GemmCommon &c, const void *x, int x_dtype, const void *bias, int bias_dtype,
                   void *y, int y_dtype, int m, int k, int n, void *workspace, size_t workspace_bytes, void *stream)
{
    OXQ_REQUIRE(x && y, OXQ_ERR_NULL, "%s: null pointer", who);
    OXQ_REQUIRE(x_dtype == OXQ_BF16, OXQ_ERR_UNSUPPORTED, "%s: activations must be bf16", who);
    OXQ_REQUIRE(valid_dtype(y_dtype) && (!bias || valid_dtype(bias_dtype)), OXQ_ERR_UNSUPPORTED, "%s: unsupported dtype", who);
    OXQ_REQUIRE(m >= 1 && k > 0 && n > 0, OXQ_ERR_BAD_SHAPE, "%s: non-positive size", who);
    OXQ_REQUIRE(k % 8 == 0, OXQ_ERR_UNSUPPORTED, "%s: in_features (%d) must be a multiple of 8", who, k);
    const size_t need = WS_HEADER + (size_t)slab_rows(n, k) * k * 2;
    OXQ_REQUIRE(workspace != nullptr && workspace_bytes >= need, OXQ_ERR_WORKSPACE,
                "%s: workspace of %zu bytes needed, got %zu", who, need, workspace_bytes);
    OXQ_REQUIRE(aligned(workspace, 256), OXQ_ERR_BAD_ALIGN, "%s: workspace must be 256-byte aligned", who);
    c.x = x; c.bias = bias; c.y = y; c.bias_dtype = bias_dtype; c.y_dtype = y_dtype; c.m = m; c.k = k; c.n = n;
    c.flag = reinterpret_cast<int *>(workspace);
    c.slab = reinterpret_cast<__nv_bfloat16 *>(reinterpret_cast<unsigned char *>(workspace) + WS_HEADER);
    c.slab_bytes = workspace_bytes - WS_HEADER;
    c.rows = slab_rows_for_m(slab_rows(n, k), n, m);
    c.st = (cudaStream_t)stream;
    return OXQ_OK; // the flag word is sticky: only oxq_gemm_check / oxq_gemm_workspace_init clear it
}

template <typename Dequant> static int run_slabs(const GemmCommon &c, Dequant dequant)
{
    for (int n_off = 0; n_off < c.n; n_off += c.rows) {
        const int cnt = c.n - n_off < c.rows ? c.n - n_off : c.rows;
        int rc = dequant(n_off, cnt);
        if (rc) return rc;
        // bias of a column shard is indexed like the output (caller passes the full-width bias)
        rc = gemm_bf16_tn(c.x, c.slab, c.bias, c.bias_dtype, c.y, c.y_dtype, c.m, cnt, c.k, c.col_base + n_off,
                          c.ldy ? c.ldy : c.n, c.flag, c.st);
        if (rc) return rc;
    }
    return OXQ_OK;
}

} // namespace oxq

using namespace oxq;

OXQ_EXPORT size_t oxq_gemm_workspace_bytes(int n, int k)
{
    if (n <= 0 || k <= 0) return WS_HEADER;
    return WS_HEADER + (size_t)slab_rows(n, k) * k * 2;
}

OXQ_EXPORT int oxq_gemm_check(const void *workspace, void *stream)
{
    clear_error();
    OXQ_REQUIRE(workspace, OXQ_ERR_NULL, "oxq_gemm_check: null workspace");
    int flag = 0;
    OXQ_CUDA(cudaMemcpyAsync(&flag, workspace, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    OXQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (flag != 0) { // report once, then the workspace is clean again
        OXQ_CUDA(cudaMemsetAsync(const_cast<void *>(workspace), 0, WS_HEADER, (cudaStream_t)stream)); // flag and split-k tickets
        OXQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    }
    OXQ_REQUIRE(flag == 0, OXQ_ERR_DEVICE_FLAG,
                "tensor-core kernel: bounded wait %d ran out (1 = ring slot, 2 = tile data, 3 = accumulator ready, "
                "4 = accumulator free, 5 = meeting of the fold warps) in a call since the last check", flag);
    return OXQ_OK;
}

OXQ_EXPORT int oxq_gemm_workspace_init(void *workspace, void *stream)
{
    clear_error();
    OXQ_REQUIRE(workspace, OXQ_ERR_NULL, "oxq_gemm_workspace_init: null workspace");
    OXQ_CUDA(cudaMemsetAsync(workspace, 0, WS_HEADER, (cudaStream_t)stream));
    return OXQ_OK;
}

OXQ_EXPORT int oxq_awq_gemm(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                            const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y,
                            int y_dtype, int m, int k, int n, int group_size, void *workspace, size_t workspace_bytes,
                            void *stream)
{
    clear_error();
    OXQ_REQUIRE(qweight && qzeros && scales, OXQ_ERR_NULL, "oxq_awq_gemm: null pointer");
    OXQ_REQUIRE(valid_dtype(scales_dtype), OXQ_ERR_UNSUPPORTED, "oxq_awq_gemm: unsupported scales dtype");
    OXQ_REQUIRE(group_size > 0 && n % 8 == 0 && k % group_size == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_awq_gemm: out_features %d must be a multiple of 8 and in_features %d a multiple of the group size %d",
                n, k, group_size);
    GemmCommon c;
    int rc = prepare("oxq_awq_gemm", c, x, x_dtype, bias, bias_dtype, y, y_dtype, m, k, n, workspace, workspace_bytes, stream);
    if (rc) return rc;
    // Up to 256 tokens: unpack inside the tensor-core kernel, no dense copy of the weight.
    if (awq_fused_supported(m, k, n, group_size, scales_dtype, x, qweight, scales))
    {
        rc = awq_fused_matmul(x, qweight, qzeros, scales, scales_dtype, bias, bias_dtype, y, y_dtype, m, k, n, group_size, 0, n, c.flag,
                              c.st, 0, 0, c.slab, c.slab_bytes);
        if (rc != OXQ_ERR_UNSUPPORTED) return rc;
    }
    return run_slabs(c, [&](int n_off, int cnt) {
        return awq_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, c.slab, k, n, group_size, n_off, cnt, c.st);
    });
}

// Column block [rows x chunks * 16 bytes] at byte offset col_off of every row of `src` -> the same place in each peer's
// buffer. Local loads, plain 16-byte stores through the peer pointers; consecutive threads take consecutive chunks of a row.
struct PeerCopyParams {
    const unsigned char *src;
    unsigned char *dst[7];
    int n_peers, rows, chunks;
    size_t ld_bytes, col_off;
};
__global__ void __launch_bounds__(256) peer_column_copy_kernel(const PeerCopyParams p)
{
    const size_t total = (size_t)p.rows * p.chunks;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / p.chunks, c = idx - r * p.chunks;
        const size_t off = r * p.ld_bytes + p.col_off + c * 16;
        const uint4 v = *reinterpret_cast<const uint4 *>(p.src + off);
        for (int pe = 0; pe < p.n_peers; pe++) *reinterpret_cast<uint4 *>(p.dst[pe] + off) = v;
    }
}

OXQ_EXPORT int oxq_awq_gemm_tp(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                               const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y,
                               void *const *y_peers, int n_peers, int y_dtype, int m, int k, int n_local, int col_base,
                               int n_full, int group_size, void *workspace, size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(qweight && qzeros && scales, OXQ_ERR_NULL, "oxq_awq_gemm_tp: null pointer");
    OXQ_REQUIRE(valid_dtype(scales_dtype), OXQ_ERR_UNSUPPORTED, "oxq_awq_gemm_tp: unsupported scales dtype");
    OXQ_REQUIRE(group_size > 0 && n_local % 8 == 0 && k % group_size == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_awq_gemm_tp: shard width %d must be a multiple of 8 and in_features %d a multiple of the group size %d",
                n_local, k, group_size);
    OXQ_REQUIRE(col_base >= 0 && n_full > 0 && col_base + n_local <= n_full, OXQ_ERR_BAD_SHAPE,
                "oxq_awq_gemm_tp: columns [%d, %d) do not lie inside an output of width %d", col_base, col_base + n_local, n_full);
    OXQ_REQUIRE(n_peers >= 0 && n_peers <= 7 && (n_peers == 0 || y_peers != nullptr), OXQ_ERR_UNSUPPORTED,
                "oxq_awq_gemm_tp: between 0 and 7 peer outputs");
    for (int i = 0; i < n_peers; i++) OXQ_REQUIRE(y_peers[i] != nullptr, OXQ_ERR_NULL, "oxq_awq_gemm_tp: null peer output %d", i);
    GemmCommon c;
    int rc = prepare("oxq_awq_gemm_tp", c, x, x_dtype, bias, bias_dtype, y, y_dtype, m, k, n_local, workspace, workspace_bytes, stream);
    if (rc) return rc;
    c.col_base = col_base; c.ldy = n_full;
    rc = OXQ_ERR_UNSUPPORTED;
    if (awq_fused_supported(m, k, n_local, group_size, scales_dtype, x, qweight, scales)) // decode-sized batches: no slab
        rc = awq_fused_matmul(x, qweight, qzeros, scales, scales_dtype, bias, bias_dtype, y, y_dtype, m, k, n_local, group_size,
                              col_base, n_full, c.flag, c.st, 0, 0, c.slab, c.slab_bytes);
    if (rc == OXQ_ERR_UNSUPPORTED)
        rc = run_slabs(c, [&](int n_off, int cnt) {
            return awq_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, c.slab, k, n_local, group_size, n_off, cnt, c.st);
        });
    if (rc || n_peers == 0) return rc;
    // The finished column block goes to the same place in every peer's output: long contiguous runs (a row of the
    // block) in 16-byte stores. Stores from the GEMM's epilogue (64-byte pieces per thread) were tried first and
    // moved only about 170 GB/s over NVLink.
    const size_t es = dtype_size(y_dtype);
    OXQ_REQUIRE(((size_t)col_base * es) % 16 == 0 && ((size_t)n_local * es) % 16 == 0 && ((size_t)n_full * es) % 16 == 0 &&
                    aligned(y, 16),
                OXQ_ERR_BAD_ALIGN, "oxq_awq_gemm_tp: the column block and the rows of y must be 16-byte aligned");
    PeerCopyParams pc;
    pc.src = reinterpret_cast<const unsigned char *>(y);
    pc.n_peers = n_peers;
    for (int i = 0; i < 7; i++) pc.dst[i] = i < n_peers ? reinterpret_cast<unsigned char *>(y_peers[i]) : nullptr;
    for (int i = 0; i < n_peers; i++) OXQ_REQUIRE(aligned(y_peers[i], 16), OXQ_ERR_BAD_ALIGN, "oxq_awq_gemm_tp: peer output %d not 16-byte aligned", i);
    pc.rows = m; pc.ld_bytes = (size_t)n_full * es; pc.col_off = (size_t)col_base * es; pc.chunks = (int)((size_t)n_local * es / 16);
    peer_column_copy_kernel<<<sm_count() * 4, 256, 0, c.st>>>(pc);
    OXQ_LAUNCH_CHECK("peer_column_copy_kernel");
    return OXQ_OK;
}

OXQ_EXPORT int oxq_gptq_gemm(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                             const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y,
                             int y_dtype, int m, int k, int n, int group_size, int bits, int sym, void *workspace,
                             size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(qweight && scales, OXQ_ERR_NULL, "oxq_gptq_gemm: null pointer");
    OXQ_REQUIRE(valid_dtype(scales_dtype), OXQ_ERR_UNSUPPORTED, "oxq_gptq_gemm: unsupported scales dtype");
    OXQ_REQUIRE(bits == 4 || bits == 8, OXQ_ERR_UNSUPPORTED, "dequantize_gptq: only 4/8-bit supported, got %d", bits);
    const int pf = 32 / bits;
    OXQ_REQUIRE(group_size > 0 && n % pf == 0 && k % pf == 0 && k % group_size == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_gptq_gemm: shape [%d, %d] incompatible with pack factor %d / group size %d", n, k, pf, group_size);
    const int use_sym = (sym != 0 || qzeros == nullptr) ? 1 : 0;
    GemmCommon c;
    int rc = prepare("oxq_gptq_gemm", c, x, x_dtype, bias, bias_dtype, y, y_dtype, m, k, n, workspace, workspace_bytes, stream);
    if (rc) return rc;
    // 4-bit, up to 256 tokens: unpack inside the tensor-core kernel (the same kernel as AWQ with the K-major operand).
    if (bits == 4 && (use_sym || aligned(qzeros, 16)) &&
        awq_fused_supported(m, k, n, group_size, scales_dtype, x, qweight, scales))
    {
        rc = awq_fused_matmul(x, qweight, use_sym ? nullptr : qzeros, scales, scales_dtype, bias, bias_dtype, y, y_dtype, m, k, n,
                              group_size, 0, n, c.flag, c.st, 1, use_sym, c.slab, c.slab_bytes);
        if (rc != OXQ_ERR_UNSUPPORTED) return rc;
    }
    return run_slabs(c, [&](int n_off, int cnt) {
        return gptq_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, c.slab, k, n, group_size, bits, use_sym,
                                      n_off, cnt, c.st);
    });
}

OXQ_EXPORT int oxq_w8a16_gemm(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                              const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y,
                              int y_dtype, int m, int k, int n, int group_size, void *workspace, size_t workspace_bytes,
                              void *stream)
{
    clear_error();
    OXQ_REQUIRE(qweight && qzeros && scales, OXQ_ERR_NULL, "oxq_w8a16_gemm: null pointer");
    OXQ_REQUIRE(valid_dtype(scales_dtype), OXQ_ERR_UNSUPPORTED, "oxq_w8a16_gemm: unsupported scales dtype");
    OXQ_REQUIRE(group_size > 0 && n % 4 == 0 && k % group_size == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_w8a16_gemm: out_features %d must be a multiple of 4 and in_features %d a multiple of the group size %d",
                n, k, group_size);
    GemmCommon c;
    int rc = prepare("oxq_w8a16_gemm", c, x, x_dtype, bias, bias_dtype, y, y_dtype, m, k, n, workspace, workspace_bytes, stream);
    if (rc) return rc;
    return run_slabs(c, [&](int n_off, int cnt) {
        return w8a16_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, c.slab, k, n, group_size, n_off, cnt, c.st);
    });
}

OXQ_EXPORT int oxq_gguf_gemm(int ggml_type, const void *x, int x_dtype, const void *blocks, const void *bias,
                             int bias_dtype, void *y, int y_dtype, int m, int k, int n, void *workspace,
                             size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(blocks, OXQ_ERR_NULL, "oxq_gguf_gemm: null pointer");
    int bel, bby;
    OXQ_REQUIRE(gguf_block_layout_host(ggml_type, bel, bby), OXQ_ERR_UNSUPPORTED, "unsupported GGML type %d", ggml_type);
    OXQ_REQUIRE(k > 0 && k % bel == 0, OXQ_ERR_BAD_SHAPE, "GGUF in_features %d is not a multiple of the block size %d", k, bel);
    OXQ_REQUIRE(aligned(blocks, 2), OXQ_ERR_BAD_ALIGN, "GGUF blocks must be 2-byte aligned");
    GemmCommon c;
    int rc = prepare("oxq_gguf_gemm", c, x, x_dtype, bias, bias_dtype, y, y_dtype, m, k, n, workspace, workspace_bytes, stream);
    if (rc) return rc;
    return run_slabs(c, [&](int n_off, int cnt) {
        return gguf_dequant_rows_bf16(ggml_type, (const uint8_t *)blocks, c.slab, k, n_off, cnt, c.st);
    });
}

OXQ_EXPORT int oxq_fp8_gemm(const void *x, int x_dtype, const uint8_t *weight, const float *scale_inv, int s_out,
                            int s_in, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                            void *workspace, size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(weight, OXQ_ERR_NULL, "oxq_fp8_gemm: null pointer");
    OXQ_REQUIRE(aligned(weight, 4), OXQ_ERR_BAD_ALIGN, "FP8 weight must be 4-byte aligned");
    int bo = n > 0 ? n : 1, bi = k > 0 ? k : 1;
    if (scale_inv) {
        OXQ_REQUIRE(s_out > 0 && s_in > 0 && n % s_out == 0 && k % s_in == 0, OXQ_ERR_BAD_SHAPE,
                    "block-wise FP8 weight_scale_inv [%d, %d] does not tile weight [%d, %d] evenly", s_out, s_in, n, k);
        bo = n / s_out;
        bi = k / s_in;
    }
    GemmCommon c;
    int rc = prepare("oxq_fp8_gemm", c, x, x_dtype, bias, bias_dtype, y, y_dtype, m, k, n, workspace, workspace_bytes, stream);
    if (rc) return rc;
    // Up to 256 tokens: widen the bytes inside the tensor-core kernel, no dense copy of the weight.
    if (fp8_fused_supported(m, k, n, bo, bi, x, weight, scale_inv)) {
        rc = fp8_fused_matmul(x, weight, scale_inv, scale_inv ? s_in : 1, bo, bi, bias, bias_dtype, y, y_dtype, m, k, n, c.flag, c.st,
                              c.slab, c.slab_bytes);
        if (rc != OXQ_ERR_UNSUPPORTED) return rc;
    }
    return run_slabs(c, [&](int n_off, int cnt) {
        return fp8_dequant_rows_bf16(weight, scale_inv, scale_inv ? s_in : 1, bo, bi, c.slab, k, n_off, cnt, c.st);
    });
}

OXQ_EXPORT int oxq_mxfp4_gemm(const void *x, int x_dtype, const uint8_t *blocks, const uint8_t *scales,
                              const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                              void *workspace, size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(blocks && scales, OXQ_ERR_NULL, "oxq_mxfp4_gemm: null pointer");
    OXQ_REQUIRE(k > 0 && k % 32 == 0, OXQ_ERR_BAD_SHAPE, "MXFP4: cols %d must be a multiple of 32", k);
    GemmCommon c;
    int rc = prepare("oxq_mxfp4_gemm", c, x, x_dtype, bias, bias_dtype, y, y_dtype, m, k, n, workspace, workspace_bytes, stream);
    if (rc) return rc;
    return run_slabs(c, [&](int n_off, int cnt) {
        return mxfp4_dequant_rows_bf16(blocks, scales, c.slab, k, n_off, cnt, c.st);
    });
}

// ---- gated FFN projection: act(x . W_gate^T) * (x . W_up^T) on a fused AWQ [gate | up] weight ----
// Decode-sized helper: y[r, j] = act(gu[r, j]) * gu[r, inter + j] for gu bf16 [m, 2 * inter] (gate half, then up half).
__global__ void __launch_bounds__(256)
gated_act_rows_kernel(const __nv_bfloat16 *__restrict__ gu, __nv_bfloat16 *__restrict__ y, int m, int inter, int act)
{
    const size_t total = (size_t)m * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / inter, j = idx % inter;
        const float gate = __bfloat162float(gu[r * 2 * inter + j]), up = __bfloat162float(gu[r * 2 * inter + inter + j]);
        float v;
        if (act == 1) v = gate * __fdividef(1.0f, 1.0f + __expf(-gate)) * up;
        else v = 0.5f * gate * (1.0f + tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate))) * up;
        y[idx] = __float2bfloat16_rn(v);
    }
}

// ---- entry point that allocates nothing ----------------------------------------------------------
// Scratch for oxq_awq_gemm_noalloc: a fixed device array that lives in the library image, so a
// caller that must not (or cannot) call cudaMalloc still has somewhere to dequantize into.
// Every GPU that loads the library holds these bytes until the process exits.
constexpr size_t NOALLOC_SLAB_BYTES = 8u << 20;
constexpr size_t NOALLOC_SCRATCH_BYTES = WS_HEADER + NOALLOC_SLAB_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
// In host code the symbol above is only a handle; the device address is looked up once per device.
static void *g_noalloc_scratch_addr[64] = {};

extern "C" int oxq_awq_gemv(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                            int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                            int group_size, void *stream);

OXQ_EXPORT int oxq_awq_ffn_gate_up(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                                   const void *scales, int scales_dtype, int activation, void *y, int m, int k, int inter,
                                   int group_size, void *workspace, size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(qweight && qzeros && scales, OXQ_ERR_NULL, "oxq_awq_ffn_gate_up: null pointer");
    OXQ_REQUIRE(valid_dtype(scales_dtype), OXQ_ERR_UNSUPPORTED, "oxq_awq_ffn_gate_up: unsupported scales dtype");
    OXQ_REQUIRE(activation == 1 || activation == 2, OXQ_ERR_UNSUPPORTED,
                "oxq_awq_ffn_gate_up: activation %d (1 = SiLU, 2 = GeLU-tanh)", activation);
    OXQ_REQUIRE(inter > 0 && inter % 8 == 0 && group_size > 0 && k > 0 && k % group_size == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_awq_ffn_gate_up: intermediate size %d must be a multiple of 8 and in_features %d of the group size %d",
                inter, k, group_size);
    const int n = 2 * inter;
    GemmCommon c;
    int rc = prepare("oxq_awq_ffn_gate_up", c, x, x_dtype, nullptr, 0, y, OXQ_BF16, m, k, n, workspace, workspace_bytes, stream);
    if (rc) return rc;
    const size_t gu_bytes = ((size_t)m * n * 2 + 255) / 256 * 256; // scratch row block [m, 2 * inter] at the head of the slab
    auto activate = [&]() -> int {
        const int blocks = (int)(((size_t)m * inter + 255) / 256);
        gated_act_rows_kernel<<<blocks < 2368 ? blocks : 2368, 256, 0, c.st>>>(c.slab, (__nv_bfloat16 *)y, m, inter, activation);
        OXQ_LAUNCH_CHECK("gated_act_rows_kernel");
        return OXQ_OK;
    };
    if (m > 16 && gu_bytes <= c.slab_bytes && awq_fused_supported(m, k, n, group_size, scales_dtype, x, qweight, scales)) {
        // Decode batches of 17 .. 256 tokens: the kernel that unpacks inside the tensor-core loop writes the
        // row block (no dense copy of the weight); what the slab holds behind the block is its scratch.
        rc = awq_fused_matmul(x, qweight, qzeros, scales, scales_dtype, nullptr, 0, c.slab, OXQ_BF16, m, k, n, group_size, 0, n,
                              c.flag, c.st, 0, 0, (unsigned char *)c.slab + gu_bytes, c.slab_bytes - gu_bytes);
        if (rc == OXQ_OK) return activate();
        if (rc != OXQ_ERR_UNSUPPORTED) return rc;
    }
    if (m <= 32) {
        // Decode: the GEMV into the scratch row block, then the activation.
        OXQ_REQUIRE(gu_bytes <= c.slab_bytes, OXQ_ERR_WORKSPACE, "oxq_awq_ffn_gate_up: workspace slab of %zu bytes, %zu needed",
                    c.slab_bytes, gu_bytes);
        rc = oxq_awq_gemv(x, x_dtype, qweight, qzeros, scales, scales_dtype, nullptr, 0, c.slab, OXQ_BF16, m, k, n, group_size,
                          stream);
        if (rc) return rc;
        return activate();
    }
    // Prefill: gate row j and up row j of the dequantized weight are written next to each other, so that
    // every accumulator tile holds (gate, up) pairs and the activation runs in the GEMM's epilogue.
    // A slab takes the same column range [a, b) of both halves: 2 (b - a) interleaved rows.
    int pairs = slab_rows(n, k) / 2;
    if (pairs < inter) pairs = pairs / 128 * 128; // whole 256-row tiles per slab
    OXQ_REQUIRE(pairs >= 8, OXQ_ERR_WORKSPACE, "oxq_awq_ffn_gate_up: workspace slab too small for in_features %d", k);
    for (int a = 0; a < inter; a += pairs) {
        const int cnt = inter - a < pairs ? inter - a : pairs;
        rc = awq_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, c.slab, k, n, group_size, a, cnt, c.st, 2, 0);
        if (rc) return rc;
        rc = awq_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, c.slab, k, n, group_size, inter + a, cnt, c.st, 2, 1);
        if (rc) return rc;
        rc = gemm_bf16_tn(c.x, c.slab, nullptr, 0, c.y, OXQ_BF16, c.m, 2 * cnt, c.k, 2 * a, inter, c.flag, c.st, activation);
        if (rc) return rc;
    }
    return OXQ_OK;
}

OXQ_EXPORT size_t oxq_awq_gemm_noalloc_max_k(void) { return NOALLOC_SLAB_BYTES / (256 * 2); }

OXQ_EXPORT int oxq_awq_gemm_noalloc(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                                    const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y,
                                    int y_dtype, int m, int k, int n, int group_size, void *stream)
{
    clear_error();
    OXQ_REQUIRE(x && y && qweight && qzeros && scales, OXQ_ERR_NULL, "oxq_awq_gemm_noalloc: null pointer");
    OXQ_REQUIRE(x_dtype == OXQ_BF16, OXQ_ERR_UNSUPPORTED, "oxq_awq_gemm_noalloc: activations must be bf16");
    OXQ_REQUIRE(valid_dtype(scales_dtype) && valid_dtype(y_dtype) && (!bias || valid_dtype(bias_dtype)),
                OXQ_ERR_UNSUPPORTED, "oxq_awq_gemm_noalloc: unsupported dtype");
    OXQ_REQUIRE(m >= 1 && k > 0 && n > 0 && group_size > 0, OXQ_ERR_BAD_SHAPE, "oxq_awq_gemm_noalloc: non-positive size");
    OXQ_REQUIRE(n % 8 == 0 && k % group_size == 0 && k % 8 == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_awq_gemm_noalloc: out_features %d must be a multiple of 8, in_features %d of 8 and of the group size %d",
                n, k, group_size);
    // The built-in scratch must hold at least one 256-row slab of the dequantized weight.
    OXQ_REQUIRE((size_t)k <= oxq_awq_gemm_noalloc_max_k(), OXQ_ERR_WORKSPACE,
                "oxq_awq_gemm_noalloc: in_features %d exceeds the built-in scratch (max %zu); use oxq_awq_gemm with a "
                "caller workspace", k, oxq_awq_gemm_noalloc_max_k());
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    OXQ_REQUIRE(device >= 0 && device < 64, OXQ_ERR_UNSUPPORTED, "oxq_awq_gemm_noalloc: device index %d out of range", device);
    if (g_noalloc_scratch_addr[device] == nullptr) {
        // First call on this device (keep it outside any stream capture): resolve the device address.
        void *addr = nullptr;
        OXQ_CUDA(cudaGetSymbolAddress(&addr, g_noalloc_scratch));
        g_noalloc_scratch_addr[device] = addr;
    }
    unsigned char *scratch = reinterpret_cast<unsigned char *>(g_noalloc_scratch_addr[device]);
    GemmCommon c;
    c.x = x; c.bias = bias; c.y = y; c.bias_dtype = bias_dtype; c.y_dtype = y_dtype; c.m = m; c.k = k; c.n = n;
    c.flag = reinterpret_cast<int *>(scratch);
    c.slab = reinterpret_cast<__nv_bfloat16 *>(scratch + WS_HEADER);
    long long rows = (long long)(NOALLOC_SLAB_BYTES / ((size_t)k * 2)) / 256 * 256;
    c.rows = rows >= n ? n : (int)rows;
    c.st = (cudaStream_t)stream; // the slab keeps the previous call's contents and is overwritten; the flag word is sticky
    return run_slabs(c, [&](int n_off, int cnt) {
        return awq_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, c.slab, k, n, group_size, n_off, cnt, c.st);
    });
}

OXQ_EXPORT int oxq_awq_gemm_noalloc_check(void *stream)
{
    clear_error();
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    OXQ_REQUIRE(device >= 0 && device < 64 && g_noalloc_scratch_addr[device] != nullptr, OXQ_ERR_NULL,
                "oxq_awq_gemm_noalloc_check: no call of oxq_awq_gemm_noalloc has run on this device yet");
    return oxq_gemm_check(g_noalloc_scratch_addr[device], stream);
}
