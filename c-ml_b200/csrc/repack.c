/*
 * One-time weight repack, host side (C11): GGUF array-of-blocks -> two planes
 * (quants, scales) whose rows start on 16-byte boundaries, so the device can
 * stream them with 128-bit loads or bulk copies. The quantized content is not
 * touched: every byte of every block lands in exactly one place, and the
 * inverse below restores the original file bytes.
 * Block layouts: include/core/gguf_quant.h:14-31 of C-ML.
 */
#include <string.h>
#include "cmlb200.h"

void cmlb200_set_error_(const char* fmt, ...);

static int block_bytes(int type) { return type == CMLB200_Q4_0 ? 18 : type == CMLB200_Q8_0 ? 34 : 0; }
static int quant_bytes(int type) { return type == CMLB200_Q4_0 ? 16 : 32; }

size_t cmlb200_qs_bytes(int type, int rows, int cols, int block) {
    (void)block;
    if (rows <= 0 || cols <= 0) return 0;
    switch (type) {
        case CMLB200_Q8_0: return (size_t)rows * (size_t)cols;
        case CMLB200_Q4_0:
        case CMLB200_NF4: return (size_t)rows * (size_t)cols / 2;
        default: return 0;
    }
}

size_t cmlb200_scale_bytes(int type, int rows, int cols, int block) {
    if (rows <= 0 || cols <= 0) return 0;
    switch (type) {
        case CMLB200_Q8_0:
        case CMLB200_Q4_0: return (size_t)rows * (size_t)(cols / 32) * 2;
        case CMLB200_NF4: return block > 0 ? (size_t)rows * (size_t)cols / (size_t)block * 4 : 0;
        default: return 0;
    }
}

static int check(int type, const void* a, const void* b, const void* c, int rows, int cols, const char* who) {
    if (!a || !b || !c) { cmlb200_set_error_("%s: NULL argument", who); return CMLB200_EINVAL; }
    if (!block_bytes(type)) { cmlb200_set_error_("%s: type %d is not a GGUF block type on this path", who, type); return CMLB200_EINVAL; }
    if (rows <= 0 || cols <= 0 || cols % 32) { cmlb200_set_error_("%s: cols (%d) must be a positive multiple of 32", who, cols); return CMLB200_EINVAL; }
    return 0;
}

int cmlb200_repack_gguf(int type, const void* h_blocks, int rows, int cols, void* h_qs, void* h_scales) {
    int rc = check(type, h_blocks, h_qs, h_scales, rows, cols, "cmlb200_repack_gguf");
    if (rc) return rc;
    const int bb = block_bytes(type), qb = quant_bytes(type);
    const size_t nblk = (size_t)rows * (size_t)(cols / 32);
    const unsigned char* src = (const unsigned char*)h_blocks;
    unsigned char* qs = (unsigned char*)h_qs;
    unsigned char* sc = (unsigned char*)h_scales;
    for (size_t b = 0; b < nblk; b++) {
        memcpy(sc + 2 * b, src + b * bb, 2);
        memcpy(qs + (size_t)qb * b, src + b * bb + 2, (size_t)qb);
    }
    return CMLB200_OK;
}

int cmlb200_unrepack_gguf(int type, const void* h_qs, const void* h_scales, int rows, int cols, void* h_blocks) {
    int rc = check(type, h_blocks, h_qs, h_scales, rows, cols, "cmlb200_unrepack_gguf");
    if (rc) return rc;
    const int bb = block_bytes(type), qb = quant_bytes(type);
    const size_t nblk = (size_t)rows * (size_t)(cols / 32);
    unsigned char* dst = (unsigned char*)h_blocks;
    const unsigned char* qs = (const unsigned char*)h_qs;
    const unsigned char* sc = (const unsigned char*)h_scales;
    for (size_t b = 0; b < nblk; b++) {
        memcpy(dst + b * bb, sc + 2 * b, 2);
        memcpy(dst + b * bb + 2, qs + (size_t)qb * b, (size_t)qb);
    }
    return CMLB200_OK;
}

int cmlb200_scales_have_subnormals(const void* h_scales_f16, size_t count) {
    const unsigned char* p = (const unsigned char*)h_scales_f16;
    if (!p) return 0;
    for (size_t i = 0; i < count; i++) {
        const unsigned h = (unsigned)p[2 * i] | ((unsigned)p[2 * i + 1] << 8);
        if ((h & 0x7C00u) == 0 && (h & 0x03FFu) != 0) return 1;
    }
    return 0;
}
