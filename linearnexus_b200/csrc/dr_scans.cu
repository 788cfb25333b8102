// Translation unit of the token-recurrent scans: the delta-rule recurrence and the RWKV-7 / RWKV-6 / Mamba-2 scans.
#include "dr_linrec.cuh"
#include "dr_recurrent.cuh"
