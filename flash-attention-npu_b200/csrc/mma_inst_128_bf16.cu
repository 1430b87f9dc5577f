#define FA_INST_HD 128
#define FA_INST_T __nv_bfloat16
#define FA_INST_NAME launch_mma_128_bf16
#define FA_INST_CONFIGS FA_MMA_CONFIGS_128
#include "mma_inst.inc"
