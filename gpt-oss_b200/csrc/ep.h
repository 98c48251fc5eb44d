// Expert parallelism over NCCL: declarations used by the C layer.
#pragma once
#include "engine.h"

namespace gptoss {
// Dispatch the routed rows of this rank's tokens to the ranks that own their
// experts, run the local experts on everything received, send the per-row
// partial sums back and add them to x.  Router results must already be in
// h->topk_i / h->topk_v.
int ep_forward(gptoss_moe *h, int layer, const void *t, void *x, int n_tokens, void *stream);
// One of the three parts of the layer over the peer-memory transport: 0 = publish,
// 1 = owner stage, 2 = combine.
int ep_forward_part(gptoss_moe *h, int layer, int part, const void *t, void *x, int n_tokens,
                    void *stream);
// NULL when the all-gathered row counts counts[src * N + dst] fit every rank's buffers.
const char *ep_counts_problem(const int *counts, int N, int max_tokens, int send_cap, int rows_cap);
void ep_destroy(gptoss_moe *h);
// 0 = rows travel with NCCL send / recv, 1 = owners and homes read each other's
// memory (ranks in separate processes of one node); -1 from the getter before
// gptoss_moe_ep_init.
int ep_set_transport(gptoss_moe *h, int transport);
int ep_get_transport(const gptoss_moe *h);
}  // namespace gptoss
