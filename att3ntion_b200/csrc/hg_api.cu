// C-ABI entry points of the three-gather hypergraph attention.
#include "att3_abi_internal.h"

extern "C" int att3_hg_forward(const void*, const void*, const void*, const void*, const void*, const void*,
                               const void*, const void*, const void*, const uint8_t*, void*, void*, void*, void*,
                               void*, void*, float*, float*, float*, float*, float*, float*, int, int, int, int, int,
                               int, int, void*) {
    return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_hg_forward: three-gather path not built");
}

extern "C" size_t att3_hg_backward_workspace_bytes(int, int, int, int) { return 0; }

extern "C" int att3_hg_backward(const void*, const void*, const void*, const void*, const void*, const void*,
                                const void*, const void*, const void*, const void*, const void*, const void*,
                                const void*, const void*, const void*, const float*, const float*, const float*,
                                const float*, const float*, const float*, const uint8_t*, void*, void*, void*, void*,
                                void*, void*, void*, void*, void*, int, int, int, int, int, int, int, void*, size_t,
                                void*) {
    return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_hg_backward: three-gather path not built");
}
