// Decode-time matrix product on packed weights: Y[m][n] = sum_k X[m][k] * W[n][k] for a small
// batch m <= 8, with W kept in its GGUF block format and decoded on the fly.  Takes over
// quantized_matmul_q4_0 / quantized_matmul_q8_0 of the reference
// (src/phfe/inference/gguf_cuda.py:299-351), which dequantise the whole weight to fp16 in HBM
// first and then call F.linear; here the packed bytes are read once (0.56 / 0.63 / 1.06 bytes per
// weight instead of 2 more written and 2 read again) and the fp16 weights exist only in registers.
//
// Each weight is decoded to exactly the fp16 value the decode kernels produce, products are
// exact in fp32 and accumulated in fp32 (mma.sync m16n8k16, f16 inputs, f32 accumulators: the
// kernel is bound by the HBM read of W, so tensor-core throughput is irrelevant), so the result
// differs from an fp32 reference only by the order of the additions.
//
// Work split: one CTA owns 16 weight rows and all of K; its 8 warps take K-chunks of 8 or 16
// blocks round-robin.  A warp stages the 16 row segments of a chunk into its own shared-memory
// ring with 16 bulk copies (one per lane) on one mbarrier, so there is no CTA-wide barrier until
// the final cross-warp reduction.
#include "common.h"
#include "dequant_kernels.cuh"

#include <atomic>

namespace pfhe {
extern std::atomic<int64_t> g_launch_count;
int status_word(int dev, int **out);        // defined in capi.cu: the pinned per-device status words
}

namespace {

using namespace pfhe;

constexpr int kGemvWarps = 8;
constexpr int kGemvStages = 2;

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Eight consecutive weights (elements 8t .. 8t+7 of the block at `blk`) as four half2, with the
// bits the decode kernels give for fp16 output.
template <int T> __device__ __forceinline__ uint4 weights8_f16(const uint8_t *blk, int t)
{
    return decode_unit<T, O_F16, O_F16, true>(blk, t);      // unit t of 4: exactly these eight elements
}

struct GemvArgs {
    const uint8_t *w;       // packed weights, 16-byte aligned, rows of (K/32)*block_bytes bytes
    const __half *x;        // [batch][ldx] activations
    void *y;                // [batch][ldy] outputs, fp32 or fp16
    int64_t rows;
    int32_t k_blocks;       // K / 32 (a multiple of 8)
    int32_t batch;          // 1..8
    int64_t ldx, ldy;
    int32_t chunk_blocks;   // 8 or 16
    int32_t y_is_f16;
    int *status;
};

template <int T>
__global__ void __launch_bounds__(kGemvWarps * 32) quant_gemv_kernel(const GemvArgs a)
{
    constexpr int BB = Fmt<T>::kBytes;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_all[kGemvWarps * kGemvStages];
    __shared__ float red[kGemvWarps][32][4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int seg_bytes = a.chunk_blocks * BB;                 // one row segment of a chunk (multiple of 16)
    const int stage_bytes = 16 * seg_bytes;
    uint8_t *ring = smem + (size_t)warp * kGemvStages * stage_bytes;
    uint64_t *full = full_all + warp * kGemvStages;
    if (lane == 0) {
        for (int s = 0; s < kGemvStages; ++s) mbar_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    const int64_t row0 = (int64_t)blockIdx.x * 16;
    const int64_t row_bytes = (int64_t)a.k_blocks * BB;
    const int n_chunks_total = (a.k_blocks + a.chunk_blocks - 1) / a.chunk_blocks;
    const int n_mine = (n_chunks_total - warp + kGemvWarps - 1) / kGemvWarps;   // chunks warp, warp+8, ...

    // lane r (< 16) copies row r's segment of chunk c into stage s
    auto issue = [&](int i) {
        const int c = warp + i * kGemvWarps;
        const int s = i % kGemvStages;
        const int b0 = c * a.chunk_blocks;
        const int nb = (a.k_blocks - b0) < a.chunk_blocks ? (a.k_blocks - b0) : a.chunk_blocks;
        const uint32_t bytes = (uint32_t)(nb * BB);             // nb is a multiple of 8: a multiple of 16 bytes
        if (lane == 0) mbar_expect_tx(&full[s], bytes * 16u);
        __syncwarp();
        if (lane < 16) {
            int64_t r = row0 + lane;
            if (r >= a.rows) r = a.rows - 1;                    // rows past the end re-read the last row; never stored
            bulk_g2s(ring + (size_t)s * stage_bytes + (size_t)lane * seg_bytes, a.w + r * row_bytes + (int64_t)b0 * BB, bytes,
                     &full[s]);
        }
    };
    for (int i = 0; i < n_mine && i < kGemvStages; ++i) issue(i);

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool has_x = g < a.batch;
    const __half *xrow = a.x + (int64_t)g * a.ldx;
    uint32_t parity_bits = 0;
    bool failed = false;
    for (int i = 0; i < n_mine; ++i) {
        const int s = i % kGemvStages;
        bool ok = true;
        if (lane == 0) ok = mbar_wait_bounded(&full[s], (parity_bits >> s) & 1u, kDeviceWaitLimitNs);
        if (__any_sync(0xffffffffu, !ok)) { failed = true; break; }
        parity_bits ^= 1u << s;

        const int c = warp + i * kGemvWarps;
        const int b0 = c * a.chunk_blocks;
        const int nb = (a.k_blocks - b0) < a.chunk_blocks ? (a.k_blocks - b0) : a.chunk_blocks;
        const uint8_t *segA = ring + (size_t)s * stage_bytes + (size_t)g * seg_bytes;
        const uint8_t *segB = segA + 8 * seg_bytes;
#pragma unroll 2
        for (int b = 0; b < nb; ++b) {
            const uint4 wa = weights8_f16<T>(segA + b * BB, t);
            const uint4 wb = weights8_f16<T>(segB + b * BB, t);
            uint4 xv = make_uint4(0u, 0u, 0u, 0u);
            if (has_x) xv = __ldg(reinterpret_cast<const uint4 *>(xrow + (int64_t)(b0 + b) * 32 + 8 * t));
            // logical k of the instruction <-> elements 8t..8t+7 of the block, the same in A and B
            const uint32_t a1[4] = {wa.x, wb.x, wa.y, wb.y};
            const uint32_t a2[4] = {wa.z, wb.z, wa.w, wb.w};
            mma_m16n8k16(acc, a1, xv.x, xv.y);
            mma_m16n8k16(acc, a2, xv.z, xv.w);
        }
        __syncwarp();
        if (i + kGemvStages < n_mine) issue(i + kGemvStages);
    }
    if (failed && lane == 0) {
        atomicExch(a.status, DEV_WAIT_TIMEOUT);
        for (int s = 0; s < kGemvStages; ++s)      // copies still in flight get a bounded chance to land
            (void)mbar_wait_bounded(&full[s], (parity_bits >> s) & 1u, kDeviceWaitLimitNs / 8);
    }

    // cross-warp reduction of the 16 x 8 tile, then one store per (row, batch column)
    red[warp][lane][0] = acc[0]; red[warp][lane][1] = acc[1]; red[warp][lane][2] = acc[2]; red[warp][lane][3] = acc[3];
    __syncthreads();
    if (warp == 0) {
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < kGemvWarps; ++w) {
            sum[0] += red[w][lane][0]; sum[1] += red[w][lane][1]; sum[2] += red[w][lane][2]; sum[3] += red[w][lane][3];
        }
        // c0: (row g, col 2t)  c1: (row g, col 2t+1)  c2: (row g+8, col 2t)  c3: (row g+8, col 2t+1); col = batch index
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t r = row0 + g + (j >> 1) * 8;
            const int m = 2 * t + (j & 1);
            if (r < a.rows && m < a.batch) {
                if (a.y_is_f16) reinterpret_cast<__half *>(a.y)[(int64_t)m * a.ldy + r] = __float2half_rn(sum[j]);
                else reinterpret_cast<float *>(a.y)[(int64_t)m * a.ldy + r] = sum[j];
            }
        }
    }
}

template <int T> int launch_gemv(const GemvArgs &a, cudaStream_t stream)
{
    const size_t smem = (size_t)kGemvWarps * kGemvStages * 16 * a.chunk_blocks * Fmt<T>::kBytes;
    auto fn = quant_gemv_kernel<T>;
    static std::atomic<unsigned long long> configured{0};          // bit per device
    int dev = 0;
    if (current_device(&dev)) return PFHE_ERR_CUDA;
    if (smem > 48 * 1024 && !(configured.load() & (1ull << dev))) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemv)");
        configured.fetch_or(1ull << dev);
    }
    const int64_t grid = (a.rows + 15) / 16;
    fn<<<(unsigned)grid, kGemvWarps * 32, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "quantized gemv launch");
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return PFHE_OK;
}

}  // namespace

extern "C" int pfhe_quantized_gemv(int ggml_type, const void *w_dev, int64_t w_bytes, int64_t rows, int64_t cols,
                                   const void *x_dev, int batch, int64_t ldx, void *y_dev, int y_dtype, int64_t ldy,
                                   void *stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int be = 0, bb = 0;
    int rc = type_geometry(ggml_type, &be, &bb);
    if (rc) return rc;
    const int base = ggml_type & ~T_ORDER_FLAG;
    if (base != T_Q4_0 && base != T_Q4_1 && base != T_Q8_0) {
        set_error("pfhe_quantized_gemv handles Q4_0, Q4_1 and Q8_0 weights, not ggml type %d", ggml_type);
        return PFHE_ERR_BAD_TYPE;
    }
    if (y_dtype != O_F32 && y_dtype != O_F16) { set_error("output dtype must be f32 or f16"); return PFHE_ERR_BAD_DTYPE; }
    if (rows < 0 || cols < 0 || batch < 1 || batch > 8 || ldx < cols || ldy < rows) {
        set_error("bad shape: rows %lld cols %lld batch %d (1..8) ldx %lld ldy %lld", (long long)rows, (long long)cols, batch,
                  (long long)ldx, (long long)ldy);
        return PFHE_ERR_BAD_ARG;
    }
    if (cols % 256) { set_error("cols must be a multiple of 256 (rows of whole 8-block groups), got %lld", (long long)cols); return PFHE_ERR_BAD_ARG; }
    const int64_t need = rows * (cols / 32) * bb;
    if (w_bytes < need) { set_error("Data too short: %lld < %lld", (long long)w_bytes, (long long)need); return PFHE_ERR_SHORT_SOURCE; }
    if (rows == 0 || cols == 0) return PFHE_OK;
    if (!w_dev || !x_dev || !y_dev) { set_error("null device pointer"); return PFHE_ERR_BAD_ARG; }
    if (reinterpret_cast<uintptr_t>(w_dev) % 16 || reinterpret_cast<uintptr_t>(x_dev) % 16 || (ldx % 8)) {
        set_error("weights and activations must be 16-byte aligned (ldx a multiple of 8)");
        return PFHE_ERR_BAD_ARG;
    }
    int dev = 0;
    if ((rc = current_device(&dev))) return rc;
    GemvArgs a;
    a.w = static_cast<const uint8_t *>(w_dev);
    a.x = static_cast<const __half *>(x_dev);
    a.y = y_dev;
    a.rows = rows;
    a.k_blocks = (int32_t)(cols / 32);
    a.batch = batch;
    a.ldx = ldx;
    a.ldy = ldy;
    a.chunk_blocks = base == T_Q8_0 ? 8 : 16;
    a.y_is_f16 = y_dtype == O_F16;
    if ((rc = status_word(dev, &a.status))) return rc;
    switch (ggml_type) {
    case T_Q4_0: return launch_gemv<T_Q4_0>(a, stream);
    case T_Q4_1: return launch_gemv<T_Q4_1>(a, stream);
    case T_Q4_0G: return launch_gemv<T_Q4_0G>(a, stream);
    case T_Q4_1G: return launch_gemv<T_Q4_1G>(a, stream);
    default: return launch_gemv<T_Q8_0>(a, stream);
    }
}
