// k_expert_tiles for IQ4_NL weights (expert_tiles.cuh).
#define EXPERT_TILES_QT moe::QT_IQ4_NL
#include "expert_tiles_inst.cuh"
