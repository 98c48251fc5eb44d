#include "ep.h"
namespace gptoss {
int ep_forward(gptoss_moe *h, int, const void *, void *, int, void *) {
  h->err = "expert parallelism is not set up: call gptoss_moe_ep_init first";
  return GPTOSS_E_STATE;
}
void ep_destroy(gptoss_moe *) {}
}  // namespace gptoss
extern "C" {
int gptoss_moe_ep_unique_id(void *) { return GPTOSS_E_STATE; }
int gptoss_moe_ep_init(gptoss_moe_t *, const void *) { return GPTOSS_E_STATE; }
}
