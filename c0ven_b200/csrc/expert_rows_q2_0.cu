// k_expert_rows for Q2_0 weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_Q2_0
#include "expert_rows_inst.cuh"
