// Library identification for the C ABI.
#include "../../include/warp34_b200.h"

extern "C" const char* warp34_b200_version(void) { return "warp34_b200 0.1 sm_100a"; }

// Bounds-checked build (-DW34_BOUNDS): the two kernel units keep a violation record each.
#ifdef W34_BOUNDS
namespace w34 {
int bounds_fetch_append(int32_t* out, int reset);
int bounds_fetch_attention(int32_t* out, int reset);
int bounds_set_pages_append(int pages);
int bounds_set_pages_attention(int pages);
}  // namespace w34
#endif

extern "C" int warp34_bounds_set_pool_pages(int32_t num_pages) {
#ifdef W34_BOUNDS
    if (num_pages < 0) return 1;
    return (w34::bounds_set_pages_append(num_pages) | w34::bounds_set_pages_attention(num_pages)) ? 1 : 0;
#else
    (void)num_pages;
    return 801;
#endif
}

extern "C" int warp34_bounds_report(int32_t* out4, int32_t reset) {
#ifdef W34_BOUNDS
    if (out4 == nullptr) return 1;
    int32_t a[4], b[4];
    if (w34::bounds_fetch_append(a, reset) || w34::bounds_fetch_attention(b, reset)) return 1;
    const int32_t* first = a[3] > 0 ? a : b;
    out4[0] = first[0];
    out4[1] = first[1];
    out4[2] = first[2];
    out4[3] = a[3] + b[3];
    return 0;
#else
    (void)out4;
    (void)reset;
    return 801;
#endif
}
