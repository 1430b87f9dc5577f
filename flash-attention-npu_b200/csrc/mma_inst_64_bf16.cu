#define FA_INST_HD 64
#define FA_INST_T __nv_bfloat16
#define FA_INST_NAME launch_mma_64_bf16
#define FA_INST_CONFIGS FA_MMA_CONFIGS_64
#include "mma_inst.inc"
