#define FA_INST_HD 256
#define FA_INST_T __nv_bfloat16
#define FA_INST_NAME launch_mma_256_bf16
#define FA_INST_CONFIGS FA_MMA_CONFIGS_256
#include "mma_inst.inc"
