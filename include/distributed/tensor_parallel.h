/* C-ML's include/distributed/tensor_parallel.h, served by libcml_b200: the fp32 sharding helpers and the column / row parallel Linear are declared in cml_quant_api.h. */
#ifndef CML_B200_DISTRIBUTED_TENSOR_PARALLEL_H
#define CML_B200_DISTRIBUTED_TENSOR_PARALLEL_H
#include "../cml_quant_api.h"
#endif
