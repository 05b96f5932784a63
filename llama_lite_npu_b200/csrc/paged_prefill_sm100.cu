// placeholder until the tcgen05 kernel lands
#include "b200kv.h"
#include "launch.h"
namespace b200kv {
int paged_prefill(const PrefillArgs&, cudaStream_t) { return B200KV_EUNSUPPORTED; }
}
