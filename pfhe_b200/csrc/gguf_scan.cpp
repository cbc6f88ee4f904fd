// Host-side helper for the GGUF header parser: walks an array of
// length-prefixed strings (u64 little-endian length, then the bytes), which is
// a dependent chain that cannot be vectorised in NumPy.  The Python parser
// (reference: _read_string / _read_metadata_value, gguf_loader.py:236-273)
// keeps its semantics; this only finds where each string starts.
#include <stdint.h>
#include <string.h>

#include "../../include/pfhe_b200.h"

extern "C" int64_t pfhe_scan_string_array(const void *base, int64_t avail, int64_t count, int64_t *offsets,
                                          int64_t *lengths)
{
    if (!base || avail < 0 || count < 0 || (count > 0 && (!offsets || !lengths))) return PFHE_ERR_BAD_ARG;
    const uint8_t *p = static_cast<const uint8_t *>(base);
    int64_t pos = 0;
    for (int64_t i = 0; i < count; ++i) {
        if (pos + 8 > avail) return PFHE_ERR_SHORT_SOURCE;
        uint64_t n;
        memcpy(&n, p + pos, 8);                       // little-endian hosts only (as the CUDA toolchain's are)
        pos += 8;
        if (n > (uint64_t)(avail - pos)) return PFHE_ERR_SHORT_SOURCE;
        offsets[i] = pos;
        lengths[i] = (int64_t)n;
        pos += (int64_t)n;
    }
    return pos;
}
