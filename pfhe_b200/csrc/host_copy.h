// Copy into pinned staging memory (see host_copy.cpp).
#pragma once

#include <stddef.h>
#include <stdint.h>

namespace pfhe {
// streaming: use non-temporal stores where the CPU has them.
void copy_to_pinned(void *dst, const void *src, size_t n, bool streaming);
}  // namespace pfhe
