// Staged decode-side kernels (shared-memory ring fed by bulk async copies, pair-symbol decode
// table).  Placeholder: declines every request so that the generic path runs.
#pragma once

#include "bhi_common.cuh"

namespace bhi {

constexpr int kStagedDeclined = -1;

template <class Codec>
static int staged_gemv(const Layer &, const typename Codec::Args &, const uint16_t *, uint16_t *, int, cudaStream_t) {
    return kStagedDeclined;
}

template <class Codec>
static int staged_decode(const Layer &, const typename Codec::Args &, uint16_t *, cudaStream_t) {
    return kStagedDeclined;
}

}  // namespace bhi
