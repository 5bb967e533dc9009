// k_expert_tiles for Q6_K weights (expert_tiles.cuh).
#define EXPERT_TILES_QT moe::QT_Q6_K
#include "expert_tiles_inst.cuh"
