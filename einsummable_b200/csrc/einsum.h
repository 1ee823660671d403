// Host-side einsummable descriptor: validation, merge_adjacent_dims, the
// structural predicates the kernel planner needs, and per-mode strides.
//
// Mirrors the parts of einsummable_t (src/einsummable/einsummable.h:8-31) that
// the reference's kernel manager consults in build()
// (src/engine/gpu/gpu_kernel_manager.cc:590-958).
#pragma once
#include <string>
#include <vector>

#include "common.h"
#include "scalarop.h"

namespace es {

struct einsum_t {
    std::vector<uint64_t>         join_shape;
    std::vector<std::vector<int>> inns;
    int                           out_rank = 0;
    int                           castable = ES_CASTABLE_NONE;
    scalarop_t                    join;

    static einsum_t from_desc(es_einsummable_desc_t const* desc);

    int join_rank() const { return (int)join_shape.size(); }

    // einsummable_t::merge_adjacent_dims (src/einsummable/einsummable.cc:166-218)
    einsum_t merge_adjacent_dims() const;

    // einsummable_t::str: mode m is written as letter 'a'+m, e.g. "ac,cb->ab"
    std::string str() const;

    bool has_aggregation() const { return out_rank < join_rank(); }
    bool has_broadcast() const;
    bool is_contraction() const;
    bool is_straight_elementwise() const;
    bool is_permutation() const;

    int out_dtype() const { return join.out_dtype(); }
    int inn_dtype(int k) const { return join.hole_dtypes.at(k); }

    uint64_t out_nelem() const;
    uint64_t inn_nelem(int k) const;
    uint64_t join_nelem() const;

    // Algorithmic work of one launch: every input read once at its own size plus the output
    // written once; 2 * prod(join_shape) multiply-adds for a contraction.
    uint64_t algorithmic_bytes() const;
    uint64_t algorithmic_flops() const { return 2 * join_nelem(); }

    // Element stride of every join mode inside input k (0 where the input does
    // not have the mode) and inside the output (0 for aggregated modes).
    std::vector<uint64_t> inn_strides(int k) const;
    std::vector<uint64_t> out_strides() const;

    // Cache key: structure + shape + join text + castable.
    std::string key() const;
    // "str|join_shape|out_rank|inn0;inn1"
    std::string describe() const;
};

} // namespace es
