// Error reporting, ABI version and weight-format validation shared by every entry point of libscmx.
#include <stdarg.h>
#include <string.h>
#include "scmx_common.cuh"

namespace scmx {

static thread_local char g_err[512] = "no error";
int g_use_pdl = 1;
unsigned long long g_wait_limit_ns = 2000000000ull;
static int32_t* g_status_word[64] = {};

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    return dev;
}
int sm_count() {
    static int n[64] = {};
    const int dev = current_device();
    if (dev < 0) return 148;
    if (!n[dev]) {
        if (cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n[dev] <= 0) n[dev] = 148;
    }
    return n[dev];
}
int32_t* device_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return g_status_word[dev];
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int make_dev_format(const scmx_format* fmt, DevFormat* out) {
    SCMX_REQUIRE(fmt != nullptr, SCMX_EINVAL, "format is NULL");
    SCMX_REQUIRE(fmt->block >= 8 && fmt->block % 8 == 0, SCMX_EFORMAT, "format.block=%d must be a multiple of 8",
                 fmt->block);
    SCMX_REQUIRE(fmt->bc_bits == 1 || fmt->bc_bits == 2 || fmt->bc_bits == 4 || fmt->bc_bits == 8, SCMX_EFORMAT,
                 "format.bc_bits=%d must be 1, 2, 4 or 8", fmt->bc_bits);
    SCMX_REQUIRE(fmt->n_mult >= 1 && fmt->n_mult <= 16 && fmt->n_mult <= (1 << fmt->bc_bits), SCMX_EFORMAT,
                 "format.n_mult=%d does not fit %d-bit block codes (max 16)", fmt->n_mult, fmt->bc_bits);
    int cmax = 0, mmax = 0;
    for (int i = 0; i < 8; ++i) {
        SCMX_REQUIRE(fmt->code_mag[i] >= 0, SCMX_EFORMAT, "negative code magnitude");
        cmax = fmt->code_mag[i] > cmax ? fmt->code_mag[i] : cmax;
    }
    for (int i = 0; i < fmt->n_mult; ++i) {
        SCMX_REQUIRE(fmt->mult[i] >= 1, SCMX_EFORMAT, "block multiplier must be >= 1");
        mmax = fmt->mult[i] > mmax ? fmt->mult[i] : mmax;
    }
    SCMX_REQUIRE(cmax * mmax <= 127, SCMX_EFORMAT, "max(code_mag) * max(mult) = %d does not fit INT8", cmax * mmax);
    memset(out, 0, sizeof(*out));
    for (int i = 0; i < 4; ++i) {
        out->mag_lo |= (uint32_t)fmt->code_mag[i] << (8 * i);
        out->mag_hi |= (uint32_t)fmt->code_mag[4 + i] << (8 * i);
        out->neg_lo |= ((uint32_t)(-fmt->code_mag[i]) & 0xFFu) << (8 * i);
        out->neg_hi |= ((uint32_t)(-fmt->code_mag[4 + i]) & 0xFFu) << (8 * i);
    }
    for (int i = 0; i < 16; ++i) out->mult4[i / 4] |= (uint32_t)(i < fmt->n_mult ? fmt->mult[i] : 1) << (8 * (i % 4));
    out->block = fmt->block;
    out->bc_bits = fmt->bc_bits;
    out->blocks_per_byte = 8 / fmt->bc_bits;
    out->block_shift = -1;
    for (int sft = 3; sft < 20; ++sft)
        if (fmt->block == (1 << sft)) out->block_shift = sft;
    out->pb_shift = fmt->bc_bits == 1 ? 3 : fmt->bc_bits == 2 ? 2 : fmt->bc_bits == 4 ? 1 : 0;
    out->pb_mask = out->blocks_per_byte - 1;
    out->bc_shift = fmt->bc_bits == 1 ? 0 : fmt->bc_bits == 2 ? 1 : fmt->bc_bits == 4 ? 2 : 3;
    out->bc_mask = (1u << fmt->bc_bits) - 1u;
    out->pow2 = 1;
    for (int i = 0; i < fmt->n_mult; ++i)
        if (fmt->mult[i] != (1 << i)) out->pow2 = 0;
    return SCMX_OK;
}

}  // namespace scmx

extern "C" const char* scmx_last_error_string(void) { return scmx::g_err; }
extern "C" int scmx_abi_version(void) { return 1; }
extern "C" int scmx_set_wait_limit_ns(unsigned long long ns) {
    SCMX_REQUIRE(ns >= 1000ull && ns <= 60000000000ull, SCMX_EINVAL, "set_wait_limit_ns: %llu outside 1 us .. 60 s", ns);
    scmx::g_wait_limit_ns = ns;
    return SCMX_OK;
}
extern "C" int scmx_set_status_word(int32_t* status) {
    int dev = 0;
    SCMX_CUDA_OK(cudaGetDevice(&dev));
    SCMX_REQUIRE(dev >= 0 && dev < 64, SCMX_ELIMIT, "device ordinal %d out of range", dev);
    scmx::g_status_word[dev] = status;
    return SCMX_OK;
}
extern "C" int scmx_set_pdl(int enable) {
    scmx::g_use_pdl = enable ? 1 : 0;
    return SCMX_OK;
}
