// Umbrella header, as include/atb/atb_infer.h of the reference.
#ifndef ATB_INFER_H
#define ATB_INFER_H
#include "atb/context.h"
#include "atb/infer_op_params.h"
#include "atb/operation.h"
#include "atb/svector.h"
#include "atb/types.h"
#include "atb/utils.h"
#endif
