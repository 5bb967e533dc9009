// k_expert_rows for IQ3_S weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_IQ3_S
#include "expert_rows_inst.cuh"
