/*
 * A C99 embedder of the library: nothing but include/pfhe_b200.h and the CUDA runtime's C API.
 * It stages seeded packed blocks from ordinary host memory through the staged loader and through
 * the no-allocation entry point, reads the decoded tensors back and compares them bit for bit with
 * the CPU oracle (oracle/dequant_oracle.c, linked in by the test that builds this file).
 * Exit status 0 and a final line "c_embedder ok: N comparisons" on success.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_runtime_api.h>

#include "pfhe_b200.h"

/* the oracle's entry points (test infrastructure) */
int64_t oracle_nbytes(int ggml_type, int64_t numel);
int oracle_read_tensor(int ggml_type, const uint8_t *src, int64_t src_bytes, int64_t numel, int out_dtype, void *out,
                       float *scratch, int n_threads);

static uint64_t rng_state = 0x9E3779B97F4A7C15ull;
static uint32_t rng_next(void)
{
    rng_state ^= rng_state << 13;
    rng_state ^= rng_state >> 7;
    rng_state ^= rng_state << 17;
    return (uint32_t)(rng_state >> 32);
}

/* Random bytes with every fp16 field replaced by a finite scale of modest size (exponent 1..20). */
static void fill_blocks(int ggml_type, uint8_t *buf, int64_t nbytes)
{
    int64_t i;
    int block = ggml_type == 2 ? 18 : (ggml_type == 3 ? 20 : 34);
    int halves = ggml_type == 3 ? 2 : 1;
    for (i = 0; i < nbytes; ++i) buf[i] = (uint8_t)rng_next();
    for (i = 0; i + block <= nbytes; i += block) {
        int h;
        for (h = 0; h < halves; ++h) {
            uint32_t r = rng_next();
            uint16_t bits = (uint16_t)((r & 0x8000u) | ((1u + (r >> 8) % 20u) << 10) | (r & 0x3FFu));
            buf[i + 2 * h] = (uint8_t)(bits & 0xFF);
            buf[i + 2 * h + 1] = (uint8_t)(bits >> 8);
        }
    }
}

#define CHECK_CUDA(call)                                                                       \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) { fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_)); return 2; } \
    } while (0)
#define CHECK_PFHE(call)                                                                       \
    do {                                                                                       \
        int rc_ = (call);                                                                      \
        if (rc_ != PFHE_OK) { fprintf(stderr, "%s: %d %s\n", #call, rc_, pfhe_last_error_string()); return 3; } \
    } while (0)

int main(void)
{
    static const int types[3] = {2, 3, 8};                       /* Q4_0, Q4_1, Q8_0 */
    static const int outs[3] = {PFHE_OUT_F32, PFHE_OUT_F16, PFHE_OUT_BF16};
    static const int64_t sizes[4] = {32, 1000, 4096 * 33, 3 * 1024 * 1024 + 17};
    int comparisons = 0, ti, oi, si;
    pfhe_loader *loader = NULL;
    cudaStream_t stream;

    printf("library version %d\n", pfhe_version());
    CHECK_CUDA(cudaSetDevice(0));
    CHECK_CUDA(cudaStreamCreate(&stream));
    CHECK_PFHE(pfhe_loader_create(0, 3, 1 << 20, 2, &loader));   /* 1 MiB slots: the larger cases take several chunks */

    for (ti = 0; ti < 3; ++ti) for (oi = 0; oi < 3; ++oi) for (si = 0; si < 4; ++si) {
        const int t = types[ti], o = outs[oi];
        const int64_t n = sizes[si];
        const int64_t in_bytes = pfhe_tensor_nbytes(t, n);
        const int64_t out_bytes = n * (o == PFHE_OUT_F32 ? 4 : 2);
        uint8_t *packed = (uint8_t *)malloc((size_t)in_bytes);
        uint8_t *want = (uint8_t *)malloc((size_t)out_bytes), *got = (uint8_t *)malloc((size_t)out_bytes);
        float *scratch = (float *)malloc((size_t)n * 4);
        void *dst = NULL;
        int via;
        if (in_bytes != oracle_nbytes(t, n)) { fprintf(stderr, "nbytes disagree for type %d n %lld\n", t, (long long)n); return 4; }
        if (!packed || !want || !got || !scratch) return 5;
        fill_blocks(t, packed, in_bytes);
        if (oracle_read_tensor(t, packed, in_bytes, n, o, want, scratch, 1)) return 6;
        CHECK_CUDA(cudaMalloc(&dst, (size_t)out_bytes + 16));
        for (via = 0; via < 2; ++via) {
            CHECK_CUDA(cudaMemsetAsync(dst, 0xA5, (size_t)out_bytes + 16, stream));
            if (via == 0) {
                CHECK_PFHE(pfhe_loader_submit(loader, packed, in_bytes, t, o, o, dst, out_bytes, n, stream));
                CHECK_PFHE(pfhe_loader_wait(loader, 60000));
            } else {
                if (in_bytes > PFHE_NOALLOC_MAX_PACKED_BYTES) continue;
                CHECK_PFHE(pfhe_dequant_from_host_noalloc(t, o, packed, in_bytes, dst, out_bytes, n, stream));
            }
            CHECK_CUDA(cudaStreamSynchronize(stream));
            CHECK_PFHE(pfhe_device_status(0));
            CHECK_CUDA(cudaMemcpy(got, dst, (size_t)out_bytes, cudaMemcpyDeviceToHost));
            if (memcmp(got, want, (size_t)out_bytes) != 0) {
                int64_t k = 0;
                while (got[k] == want[k]) ++k;
                fprintf(stderr, "mismatch: type %d out %d n %lld via %d at byte %lld\n", t, o, (long long)n, via, (long long)k);
                return 1;
            }
            ++comparisons;
        }
        CHECK_CUDA(cudaFree(dst));
        free(packed); free(want); free(got); free(scratch);
    }
    /* the error path speaks C too */
    if (pfhe_dequant_launch(99, PFHE_OUT_F16, NULL, 0, NULL, 0, 1, NULL) != PFHE_ERR_BAD_TYPE) return 7;
    if (strlen(pfhe_last_error_string()) == 0) return 8;
    CHECK_PFHE(pfhe_loader_destroy(loader));
    CHECK_CUDA(cudaStreamDestroy(stream));
    printf("c_embedder ok: %d comparisons\n", comparisons);
    return 0;
}
