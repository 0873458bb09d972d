#define DSDPA_T float
#include "dsdpa_inst_bwd.inc"
