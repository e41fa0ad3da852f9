/*
 * pulp_train.h - umbrella header under the name that PULP-TrainLib user code and
 * TrainLib_Deployer-generated code include (reference: lib/include/pulp_train.h).
 * It pulls in the runtime stand-in, the ABI-identical structs and prototypes of the
 * training-step primitives, and this library's own extensions.
 */
#ifndef PULP_TRAIN_H
#define PULP_TRAIN_H
#include "pmsis.h"
#include "trainlib_b200_abi.h"
#include "trainlib_b200.h"
#endif
