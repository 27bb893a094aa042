// Umbrella header of the libraries that sit beside the core, collectives and EP headers.
#ifndef TILEXR_EXTRAS_H
#define TILEXR_EXTRAS_H

#include "tilexr_fused.h"
#include "tilexr_hostsim.h"
#include "tilexr_moonep.h"
#include "tilexr_moonep_combine_v2.h"
#include "tilexr_moonep_trace.h"
#include "tilexr_probes.h"
#include "../checker/checker.h"

#endif
