// k_expert_tiles for IQ3_XXS weights (expert_tiles.cuh).
#define EXPERT_TILES_QT moe::QT_IQ3_XXS
#include "expert_tiles_inst.cuh"
