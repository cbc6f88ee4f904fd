// Host-side copy of packed bytes into pinned staging memory.
//
// The destination is written once and then read only by the GPU's copy
// engine, so on x86-64 with AVX2 the copy uses non-temporal stores: the
// destination lines are not read for ownership and do not displace the page
// cache lines still to be read.  Elsewhere it is memcpy.
#include "host_copy.h"

#include <string.h>

#if defined(__x86_64__) && defined(__GNUC__)
#include <immintrin.h>

namespace {

__attribute__((target("avx2"))) void copy_nt_avx2(uint8_t *dst, const uint8_t *src, size_t n)
{
    // Head: bring dst to a 32-byte boundary.
    const size_t head = (32 - (reinterpret_cast<uintptr_t>(dst) & 31)) & 31;
    if (head) {
        const size_t h = head < n ? head : n;
        memcpy(dst, src, h);
        dst += h; src += h; n -= h;
    }
    while (n >= 128) {
        const __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(src));
        const __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(src + 32));
        const __m256i c = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(src + 64));
        const __m256i d = _mm256_loadu_si256(reinterpret_cast<const __m256i *>(src + 96));
        _mm256_stream_si256(reinterpret_cast<__m256i *>(dst), a);
        _mm256_stream_si256(reinterpret_cast<__m256i *>(dst + 32), b);
        _mm256_stream_si256(reinterpret_cast<__m256i *>(dst + 64), c);
        _mm256_stream_si256(reinterpret_cast<__m256i *>(dst + 96), d);
        src += 128; dst += 128; n -= 128;
    }
    _mm_sfence();
    if (n) memcpy(dst, src, n);
}

bool have_avx2()
{
    static const bool ok = __builtin_cpu_supports("avx2");
    return ok;
}

}  // namespace

namespace pfhe {
void copy_to_pinned(void *dst, const void *src, size_t n, bool streaming)
{
    if (streaming && n >= 4096 && have_avx2())
        copy_nt_avx2(static_cast<uint8_t *>(dst), static_cast<const uint8_t *>(src), n);
    else
        memcpy(dst, src, n);
}
}  // namespace pfhe

#else

namespace pfhe {
void copy_to_pinned(void *dst, const void *src, size_t n, bool) { memcpy(dst, src, n); }
}  // namespace pfhe

#endif
