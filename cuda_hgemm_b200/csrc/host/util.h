// Small helpers of the driver: ceiling division and the SM-version tables used for the
// device banner (reference src/common/util.h:11-72, whose tables stop at 9.0; 10.x is added).
#pragma once

#include <stddef.h>

#include "cuda_runtime_api.h"

inline __host__ __device__ size_t div_ceil(size_t a, size_t b) {
    return (a + b - 1) / b;
}

// FP32 CUDA cores per SM for a compute capability; 0 when unknown.
inline int convert_SM_to_cores(int major, int minor) {
    switch ((major << 4) | minor) {
        case 0x30: case 0x32: case 0x35: case 0x37: return 192;
        case 0x50: case 0x52: case 0x53: return 128;
        case 0x60: return 64;
        case 0x61: case 0x62: return 128;
        case 0x70: case 0x72: case 0x75: case 0x80: return 64;
        case 0x86: case 0x87: case 0x89: case 0x90: return 128;
        case 0xa0: case 0xa1: case 0xa3: return 128;
        case 0xc0: case 0xc1: return 128;
        default: return 0;
    }
}

inline const char *convert_SM_to_arch_name(int major, int minor) {
    switch (major) {
        case 3: return "Kepler";
        case 5: return "Maxwell";
        case 6: return "Pascal";
        case 7: return minor == 0 ? "Volta" : (minor == 2 ? "Xavier" : "Turing");
        case 8: return minor == 9 ? "Ada" : "Ampere";
        case 9: return "Hopper";
        case 10: case 12: return "Blackwell";
        default: return "Graphics Device";
    }
}
