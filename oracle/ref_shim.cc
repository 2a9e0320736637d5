// Shim that lets the reference's own host checkers be compiled with g++ and called from C.
// TEST INFRASTRUCTURE ONLY (same rule as the rest of this directory).
//
// The functions themselves are NOT in this file.  ref_build.py cuts them, unmodified, out of the reference
// checkout (opus_gemm/gemm_a8w8_8wave.cc, opus_gemm/block_scale_gemm/gemm_a8w8_blockscale_host.cc,
// opus_fmm/flatmm_a8w8_gfx950.cc, opus_gemm/gemm_a16w16_8wave.cc, opus_fmm/flatmm_a16w16_gfx950.cc) into
// *.inc files of a scratch directory and this file includes them, each set inside its own namespace.  What the
// shim supplies is only what those lines expect from headers that do not exist here:
//   host_fp8_t         __hip_fp8_e4m3 (ROCm hip/hip_fp8.h, third party) -> NVIDIA's host __nv_fp8_e4m3, the same
//                      OCP E4M3 encoding with round-to-nearest-even, saturate-to-finite conversion
//   bf16_t             __bf16 (compiler builtin in both toolchains)
//   opus::get_warp_size(), opus::remove_cvref_t   the two names shuffle_b uses (a gfx9 wave has 64 lanes)
//   Traits::W_N, W_K   constants parsed from the reference's traits structs into ref_traits.inc
#include <cuda_fp8.h>

#include <algorithm>
#include <cassert>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <type_traits>
#include <omp.h>

namespace opus {
constexpr int get_warp_size() { return 64; }
template <class T>
using remove_cvref_t = std::remove_cv_t<std::remove_reference_t<T>>;
}  // namespace opus

using fp32_t = float;
using host_fp8_t = __nv_fp8_e4m3;
using bf16_t = __bf16;
static_assert(sizeof(host_fp8_t) == 1 && sizeof(bf16_t) == 2, "operand types are plain 8- and 16-bit storage");

#include "ref_traits.inc"   // struct fmm_a8w8_traits { W_N, W_K }; struct fmm_a16w16_traits { W_N, W_K };

namespace ref_a8w8 {
#include "a8w8_valid_vector.inc"
#include "a8w8_gemm_ref.inc"
}  // namespace ref_a8w8
namespace ref_bs {
#include "bs_valid_vector.inc"
#include "bs_gemm_ref.inc"
}  // namespace ref_bs
namespace ref_fmm {
#include "fmm_gemm_ref.inc"
#include "fmm_shuffle_b.inc"
}  // namespace ref_fmm
namespace ref_a16 {
#include "a16_gemm_ref.inc"
}  // namespace ref_a16
namespace ref_fmm16 {
#include "fmm16_gemm_ref.inc"
#include "fmm16_shuffle_b.inc"
}  // namespace ref_fmm16

static const host_fp8_t* F8(const void* p) { return reinterpret_cast<const host_fp8_t*>(p); }
static const bf16_t* B16(const void* p) { return reinterpret_cast<const bf16_t*>(p); }

extern "C" {

// static_cast<host_fp8_t>(float): what rand_vector does with every drawn value (gemm_a8w8_8wave.cc:576)
uint8_t ref_cast_e4m3(float x) {
    const host_fp8_t v = static_cast<host_fp8_t>(x);
    return *reinterpret_cast<const uint8_t*>(&v);
}
float ref_e4m3_to_f32(uint8_t b) { return static_cast<fp32_t>(*reinterpret_cast<const host_fp8_t*>(&b)); }

void ref_gemm_nt(const void* a, const void* b, float* c, int m, int n, int k, int lda, int ldb, int ldc) {
    ref_a8w8::gemm_ref(F8(a), F8(b), c, m, n, k, lda, ldb, ldc);
}
void ref_gemm_blockscale(const void* a, const void* b, const float* sfa, const float* sfb, float* c, int m, int n, int k,
                         int lda, int ldb, int ldc, int stride_sfa, int stride_sfb, int group_m, int group_n, int group_k) {
    ref_bs::gemm_ref(F8(a), F8(b), sfa, sfb, c, m, n, k, lda, ldb, ldc, stride_sfa, stride_sfb, group_m, group_n, group_k);
}
void ref_gemm_kn(const void* a, const void* b_kn, float* c, int m, int n, int k, int lda, int ldb, int ldc) {
    ref_fmm::gemm_ref(F8(a), F8(b_kn), c, m, n, k, lda, ldb, ldc);
}
void ref_shuffle_b(const void* b_kn, void* out, int n, int k) {
    ref_fmm::shuffle_b<host_fp8_t, fmm_a8w8_traits>(F8(b_kn), reinterpret_cast<host_fp8_t*>(out), n, k);
}
void ref_gemm_nt_bf16(const void* a, const void* b, void* c, int m, int n, int k, int lda, int ldb, int ldc) {
    ref_a16::gemm_ref(B16(a), B16(b), reinterpret_cast<bf16_t*>(c), m, n, k, lda, ldb, ldc);
}
void ref_gemm_kn_bf16(const void* a, const void* b_kn, void* c, int m, int n, int k, int lda, int ldb, int ldc) {
    ref_fmm16::gemm_ref(B16(a), B16(b_kn), reinterpret_cast<bf16_t*>(c), m, n, k, lda, ldb, ldc);
}
void ref_shuffle_b_bf16(const void* b_kn, void* out, int n, int k) {
    ref_fmm16::shuffle_b<bf16_t, fmm_a16w16_traits>(B16(b_kn), reinterpret_cast<bf16_t*>(out), n, k);
}
// the two copies of valid_vector (8wave and block-scale host) are exported separately
int ref_valid_vector(const float* ref, const float* res, int n, float threshold) {
    return ref_a8w8::valid_vector<float>(ref, res, n, threshold) ? 1 : 0;
}
int ref_valid_vector_bs(const float* ref, const float* res, int n, float threshold) {
    return ref_bs::valid_vector<float>(ref, res, n, threshold) ? 1 : 0;
}
int ref_fast_math(void) {
#ifdef __FAST_MATH__
    return 1;
#else
    return 0;
#endif
}
}
