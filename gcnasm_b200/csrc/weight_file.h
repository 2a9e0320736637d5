// Weight file: a pre-quantised (and optionally pre-shuffled) B operand with its scales, so that a decode run does
// not repeat the host-side layout pass the reference performs on every start (opus_fmm/flatmm_a8w8_gfx950.cc:736-742
// shuffles 132 MB on the host before the first launch).  Host code only; little-endian.
//
//   offset 0   : b200_weight_desc header, 128 bytes (magic "B200WGT1", sizes, layout and scale ids, checksum)
//   offset 128 : N*K operand bytes in the layout the header names
//   then       : padding to a multiple of 64 bytes
//   then       : scale bytes (fp32 [N/128][K/128] for block scales, E8M0 atoms for MX, one fp32 for per-tensor)
//
// The checksum is FNV-1a (64-bit) over the operand bytes followed by the scale bytes.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../../include/b200gemm.h"

namespace b200 {

static_assert(sizeof(b200_weight_desc) == 128, "the header is 128 bytes");
static const char kWeightMagic[8] = {'B', '2', '0', '0', 'W', 'G', 'T', '1'};

inline uint64_t fnv1a64(const void* p, size_t n, uint64_t h = 1469598103934665603ull) {
    const unsigned char* b = static_cast<const unsigned char*>(p);
    for (size_t i = 0; i < n; ++i) {
        h ^= b[i];
        h *= 1099511628211ull;
    }
    return h;
}

inline int64_t expected_scale_bytes(const b200_weight_desc& d) {
    switch (d.scale_mode) {
        case B200_SCALE_NONE: return 0;
        case B200_SCALE_TENSOR: return 4;
        case B200_SCALE_BLOCK: return (d.n % 128 == 0 && d.k % 128 == 0) ? 4 * (d.n / 128) * (d.k / 128) : -1;
        case B200_SCALE_MX: return d.k % 128 == 0 ? ((d.n + 127) / 128) * (d.k / 128) * 512 : -1;
        default: return -1;
    }
}

// Largest N or K a header may state: keeps n * k and every scale-size product far inside int64_t, whatever a
// corrupt or hostile file says (the fields come straight from disk).
constexpr int64_t kWeightMaxDim = int64_t(1) << 31;

inline int check_desc(const b200_weight_desc& d) {
    if (std::memcmp(d.magic, kWeightMagic, 8) != 0 || d.version != 1) return B200_ERR_BAD_ARG;
    if (d.n <= 0 || d.k <= 0 || d.n > kWeightMaxDim || d.k > kWeightMaxDim) return B200_ERR_BAD_ARG;
    if (d.b_layout != B200_B_NK_ROWMAJOR && d.b_layout != B200_B_FLAT_16x16) return B200_ERR_BAD_ARG;
    if (d.b_layout == B200_B_FLAT_16x16 && (d.n % 16 != 0 || d.k % 16 != 0)) return B200_ERR_UNSUPPORTED;
    if (d.data_bytes != d.n * d.k) return B200_ERR_BAD_ARG;
    const int64_t sb = expected_scale_bytes(d);
    if (sb < 0) return B200_ERR_UNSUPPORTED;
    if (d.scale_bytes != sb) return B200_ERR_BAD_ARG;
    return B200_OK;
}

inline int64_t scale_offset(const b200_weight_desc& d) { return 128 + (d.data_bytes + 63) / 64 * 64; }

inline int weight_file_write(const char* path, int32_t b_layout, int32_t scale_mode, int64_t n, int64_t k, const void* data,
                             const void* scales) {
    if (!path || !data) return B200_ERR_BAD_ARG;
    if (n <= 0 || k <= 0 || n > kWeightMaxDim || k > kWeightMaxDim) return B200_ERR_BAD_ARG;
    b200_weight_desc d;
    std::memset(&d, 0, sizeof(d));
    std::memcpy(d.magic, kWeightMagic, 8);
    d.version = 1;
    d.b_layout = b_layout;
    d.scale_mode = scale_mode;
    d.n = n;
    d.k = k;
    d.data_bytes = n * k;
    d.scale_bytes = expected_scale_bytes(d);
    if (d.scale_bytes < 0) return B200_ERR_UNSUPPORTED;
    int rc = check_desc(d);
    if (rc) return rc;
    if (d.scale_bytes > 0 && !scales) return B200_ERR_BAD_ARG;
    d.checksum = fnv1a64(scales, static_cast<size_t>(d.scale_bytes), fnv1a64(data, static_cast<size_t>(d.data_bytes)));
    std::FILE* f = std::fopen(path, "wb");
    if (!f) return B200_ERR_IO;
    bool ok = std::fwrite(&d, sizeof(d), 1, f) == 1;
    ok = ok && std::fwrite(data, 1, static_cast<size_t>(d.data_bytes), f) == static_cast<size_t>(d.data_bytes);
    const char zeros[64] = {0};
    const size_t pad = static_cast<size_t>(scale_offset(d) - 128 - d.data_bytes);
    ok = ok && (pad == 0 || std::fwrite(zeros, 1, pad, f) == pad);
    ok = ok && (d.scale_bytes == 0 || std::fwrite(scales, 1, static_cast<size_t>(d.scale_bytes), f) == static_cast<size_t>(d.scale_bytes));
    ok = (std::fclose(f) == 0) && ok;
    return ok ? B200_OK : B200_ERR_IO;
}

inline int weight_file_stat(const char* path, b200_weight_desc* out) {
    if (!path || !out) return B200_ERR_BAD_ARG;
    std::FILE* f = std::fopen(path, "rb");
    if (!f) return B200_ERR_IO;
    b200_weight_desc d;
    const bool got = std::fread(&d, sizeof(d), 1, f) == 1;
    long long size = -1;
    if (got && fseeko(f, 0, SEEK_END) == 0) size = static_cast<long long>(ftello(f));
    std::fclose(f);
    if (!got) return B200_ERR_IO;
    int rc = check_desc(d);
    if (rc) return rc;
    if (size >= 0 && size < scale_offset(d) + d.scale_bytes) return B200_ERR_IO;      // truncated
    *out = d;
    return B200_OK;
}

inline int weight_file_read(const char* path, void* data, size_t data_capacity, void* scales, size_t scale_capacity) {
    b200_weight_desc d;
    int rc = weight_file_stat(path, &d);
    if (rc) return rc;
    if (!data || data_capacity < static_cast<size_t>(d.data_bytes)) return B200_ERR_TOO_LARGE;
    if (d.scale_bytes > 0 && (!scales || scale_capacity < static_cast<size_t>(d.scale_bytes))) return B200_ERR_TOO_LARGE;
    std::FILE* f = std::fopen(path, "rb");
    if (!f) return B200_ERR_IO;
    bool ok = std::fseek(f, 128, SEEK_SET) == 0;
    ok = ok && std::fread(data, 1, static_cast<size_t>(d.data_bytes), f) == static_cast<size_t>(d.data_bytes);
    ok = ok && fseeko(f, static_cast<off_t>(scale_offset(d)), SEEK_SET) == 0;
    ok = ok && (d.scale_bytes == 0 || std::fread(scales, 1, static_cast<size_t>(d.scale_bytes), f) == static_cast<size_t>(d.scale_bytes));
    std::fclose(f);
    if (!ok) return B200_ERR_IO;
    const uint64_t sum = fnv1a64(scales, static_cast<size_t>(d.scale_bytes), fnv1a64(data, static_cast<size_t>(d.data_bytes)));
    return sum == d.checksum ? B200_OK : B200_ERR_CORRUPT;
}

}  // namespace b200
