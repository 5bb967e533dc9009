// k_expert_rows for Q6_K weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_Q6_K
#include "expert_rows_inst.cuh"
