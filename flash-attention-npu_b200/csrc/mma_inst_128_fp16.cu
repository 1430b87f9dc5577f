#define FA_INST_HD 128
#define FA_INST_T __half
#define FA_INST_NAME launch_mma_128_fp16
#define FA_INST_CONFIGS FA_MMA_CONFIGS_128
#include "mma_inst.inc"
