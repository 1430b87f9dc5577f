#define FA_INST_T __half
#define FA_INST_NAME launch_decode_128_fp16
#include "decode_inst.inc"
