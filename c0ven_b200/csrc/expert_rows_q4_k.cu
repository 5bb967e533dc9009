// k_expert_rows for Q4_K weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_Q4_K
#include "expert_rows_inst.cuh"
