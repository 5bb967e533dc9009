// k_expert_tiles for Q2_0 weights (expert_tiles.cuh).
#define EXPERT_TILES_QT moe::QT_Q2_0
#include "expert_tiles_inst.cuh"
