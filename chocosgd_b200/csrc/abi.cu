// ABI self-description: the Python side mirrors ChocoParams with a ctypes.Structure and
// checks these numbers at import time, so a layout drift fails loudly instead of
// corrupting a kernel launch.
#include <stddef.h>

#include "common.cuh"

extern "C" int choco_params_size() { return (int)sizeof(ChocoParams); }
extern "C" int choco_params_offset(int which) {
  switch (which) {
    case 0: return (int)offsetof(ChocoParams, outbox);
    case 1: return (int)offsetof(ChocoParams, hyper);
    case 2: return (int)offsetof(ChocoParams, wait_budget_ns);
    case 3: return (int)offsetof(ChocoParams, tab);
    case 4: return (int)offsetof(ChocoParams, w_self);
    case 5: return (int)offsetof(ChocoParams, n_peers);
    case 6: return (int)offsetof(ChocoParams, seed);
    default: return -1;
  }
}
extern "C" int choco_max_peers() { return CHOCO_MAX_PEERS; }
extern "C" int choco_hist_words() { return CHOCO_HIST_WORDS; }
