// Umbrella header of the host layer (the subset of ginn's API behind which the B200 library sits).
#ifndef GINN_B200_HOST_GINN_H
#define GINN_B200_HOST_GINN_H
#include <ginn/autobatch.h>
#include <ginn/node/affine.h>
#include <ginn/node/conv.h>
#include <ginn/node/data.h>
#include <ginn/node/lstmcell.h>
#include <ginn/node/nlnode.h>
#include <ginn/node/pick.h>
#include <ginn/node/prod.h>
#include <ginn/prod.h>
#include <ginn/update/update.h>
#endif
