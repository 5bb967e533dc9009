// k_expert_rows for IQ3_XXS weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_IQ3_XXS
#include "expert_rows_inst.cuh"
