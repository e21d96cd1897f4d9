// Error macro of the host driver (interface of the reference's bfAintBGemm/gpu_utils.hpp:5-11) over the int status
// codes of the C ABI.  The reference exits with code 0 on a failed call; this one exits non-zero.
#pragma once
#include <cstdio>
#include <cstdlib>
#include "afb_capi.h"

#define GPU_CHECK_ERROR(call)                                                                        \
    do {                                                                                             \
        const int afb_status__ = (call);                                                             \
        if (afb_status__ != AFB_OK) {                                                                \
            std::printf("[afb error](%d: %s%s%s), failed to call %s \n", afb_status__,                \
                        afb_status_string(afb_status__), afb_status__ == AFB_ERR_CUDA ? " - " : "",   \
                        afb_status__ == AFB_ERR_CUDA ? afb_last_cuda_error_string() : "", #call);     \
            std::exit(1);                                                                            \
        }                                                                                            \
    } while (0)
