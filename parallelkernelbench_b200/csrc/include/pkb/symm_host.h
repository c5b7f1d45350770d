// Host-side conversion of the C API's group descriptor into the device view used by kernels.
#pragma once
#include "pkb/collectives_api.h"
#include "pkb/host.h"
#include "pkb/symm.cuh"

namespace pkb {

inline SymmCtx symm_ctx_from_api(const pkb_symm_ctx* h) {
  SymmCtx c;
  c.base = h->base; c.stride = h->stride; c.mc_base = h->mc_base;
  c.rank = h->rank; c.world = h->world; c.gsize = h->gsize; c.grank = h->grank;
  for (int i = 0; i < kSymmMaxWorld; ++i) c.members[i] = h->members[i];
  c.channel = h->channel;
  c.status = status_block_device_ptr();
  c.budget_ns = h->budget_ns ? h->budget_ns : kDefaultWaitBudgetNs;
  return c;
}

inline int symm_ctx_check(const pkb_symm_ctx* h) {
  PKB_CHECK_ARG(h != nullptr && h->base != 0 && h->stride != 0, "symmetric heap not initialised");
  PKB_CHECK_ARG(h->gsize >= 1 && h->gsize <= kSymmMaxWorld && h->grank >= 0 && h->grank < h->gsize, "bad group");
  PKB_CHECK_ARG(h->channel >= 0 && h->channel < kSymmChannels, "bad channel");
  return kApiOk;
}

}  // namespace pkb
