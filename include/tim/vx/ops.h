// Convenience include of every op class this backend executes
// (reference: include/tim/vx/ops.h lists ~110 headers; the quantized CNN path
// needs the compute ops; Reshape, Transpose, Concat and DataConvert are what the reference's exported
// graphs put between them), and of a few that are only declared, because the reference's own layout
// inference and simple-operation tests name them.
#ifndef TIM_VX_OPS_H_
#define TIM_VX_OPS_H_
#include "tim/vx/ops/activations.h"
#include "tim/vx/ops/addn.h"
#include "tim/vx/ops/concat.h"
#include "tim/vx/ops/conv2d.h"
#include "tim/vx/ops/elementwise.h"
#include "tim/vx/ops/fullyconnected.h"
#include "tim/vx/ops/groupedconv2d.h"
#include "tim/vx/ops/instancenormalization.h"
#include "tim/vx/ops/nbg.h"
#include "tim/vx/ops/pool2d.h"
#include "tim/vx/ops/relational_operations.h"
#include "tim/vx/ops/reshape.h"
#include "tim/vx/ops/resize.h"
#include "tim/vx/ops/roi_align.h"
#include "tim/vx/ops/simple_operations.h"
#include "tim/vx/ops/softmax.h"
#include "tim/vx/ops/transpose.h"
#endif  // TIM_VX_OPS_H_
