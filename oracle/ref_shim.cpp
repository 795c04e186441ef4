/*
 * ref_shim.cpp -- C entry points around the UPSTREAM C++ core.  TEST INFRASTRUCTURE ONLY.
 *
 * oracle/build.py compiles this file together with the upstream source
 * csrc/core/turboquant_core.cpp (taken from an upstream checkout, not copied into this
 * repository) into oracle/_ref/libtq_ref.so.  The shim only forwards raw pointers to the
 * upstream functions declared in csrc/core/turboquant_core.h, feeding them the rotation
 * matrix, boundaries and centroids the caller passes, so that the upstream code runs on the
 * same constants as the kernels it is compared with (the upstream core would otherwise draw
 * its rotation from a different random generator, turboquant_core.cpp:137-213).
 */
#include <cstdint>
#include <cstring>
#include <string>

#include "turboquant_core.h"

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

__attribute__((visibility("default"))) int tqr_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

__attribute__((visibility("default"))) void tqr_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* turboquant::search_packed, csrc/core/turboquant_core.cpp:407-514 */
__attribute__((visibility("default"))) void tqr_search_packed(
    const float* queries, int nq, const uint8_t* packed, const float* norms, int n, int dim,
    int bits, const float* rotation, const float* centroids, int k, float* out_scores,
    int64_t* out_ids) {
    turboquant::search_packed(queries, nq, packed, norms, n, dim, bits, rotation, centroids, k,
                              out_scores, out_ids);
}

/* turboquant::quantize_vectors, csrc/core/turboquant_core.cpp:277-343, with caller constants */
__attribute__((visibility("default"))) void tqr_quantize(
    const float* vectors, int n, int dim, const float* rotation, const float* boundaries,
    const float* centroids, int bits, uint8_t* packed, float* norms) {
    turboquant::Codebook cb;
    cb.bits = bits;
    cb.dim = dim;
    cb.n_levels = 1 << bits;
    cb.scale = 1.0;
    cb.scaled_boundaries.assign(boundaries, boundaries + cb.n_levels - 1);
    cb.scaled_centroids.assign(centroids, centroids + cb.n_levels);
    turboquant::quantize_vectors(vectors, n, dim, rotation, cb, packed, norms);
}

/* turboquant::dequantize_vectors, csrc/core/turboquant_core.cpp:345-401 */
__attribute__((visibility("default"))) void tqr_dequantize(
    const uint8_t* packed, const float* norms, int n, int dim, const float* rotation,
    const float* centroids, int bits, float* out) {
    turboquant::Codebook cb;
    cb.bits = bits;
    cb.dim = dim;
    cb.n_levels = 1 << bits;
    cb.scale = 1.0;
    cb.scaled_boundaries.assign(cb.n_levels - 1, 0.0f);
    cb.scaled_centroids.assign(centroids, centroids + cb.n_levels);
    turboquant::dequantize_vectors(packed, norms, n, dim, rotation, cb, out);
}

/* turboquant::TurboQuantIndex add() + save(), csrc/core/turboquant_core.cpp:523-581: builds an index with
 * the core's OWN rotation and codebook (drawn from `seed` by its generators) and writes it in the core's
 * file layout; the rows the core holds are returned for comparison.  Used to produce the file fixture. */
__attribute__((visibility("default"))) int tqr_index_build_save(
    const float* vectors, int n, int dim, int bits, int seed, const char* path, uint8_t* out_packed,
    float* out_norms) {
    try {
        turboquant::TurboQuantIndex idx(dim, bits, seed);
        idx.add(vectors, n);
        idx.save(path);
        std::memcpy(out_packed, idx.packed_codes().data(), idx.packed_codes().size());
        std::memcpy(out_norms, idx.norms().data(), idx.norms().size() * sizeof(float));
        return idx.n_vectors();
    } catch (...) {
        return -1;
    }
}

}  // extern "C"
