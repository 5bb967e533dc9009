// k_expert_rows for Q8_0 weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_Q8_0
#include "expert_rows_inst.cuh"
