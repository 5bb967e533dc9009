// k_expert_rows for IQ4_NL weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_IQ4_NL
#include "expert_rows_inst.cuh"
