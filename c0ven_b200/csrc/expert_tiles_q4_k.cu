// k_expert_tiles for Q4_K weights (expert_tiles.cuh).
#define EXPERT_TILES_QT moe::QT_Q4_K
#include "expert_tiles_inst.cuh"
