// Mixture-of-experts block: internal declarations.
#pragma once
#include "nnq_internal.h"

struct nnq_moe {
    nnq_ctx *ctx;
    int n_experts, hidden, inter, top_k;
    int e_begin, e_local;  // experts held by this device: [e_begin, e_begin + e_local)
    float limit;
    int layout;            // nnq_moe_layout
    int fmt;               // nnq_format of the expert weights
    float *d_router_w, *d_router_b;
    uint8_t *d_gu, *d_gu_scales, *d_dn, *d_dn_scales;
    size_t gu_bytes, gu_scale_bytes, dn_bytes, dn_scale_bytes;   // per tensor (all experts)
    float *d_gu_bias, *d_dn_bias;
    // tiled copies of the expert weights for the grouped token-column kernel ([N, K] layouts whose
    // format and K have a tiled layout); NULL otherwise
    uint8_t *d_gu_tiled, *d_dn_tiled;
    size_t gu_tile_stride, dn_tile_stride;   // bytes per expert
};
