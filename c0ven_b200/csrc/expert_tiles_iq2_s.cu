// k_expert_tiles for IQ2_S weights (expert_tiles.cuh).
#define EXPERT_TILES_QT moe::QT_IQ2_S
#include "expert_tiles_inst.cuh"
