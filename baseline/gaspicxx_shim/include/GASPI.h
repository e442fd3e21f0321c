#pragma once
// GPI-2's C header: the reference includes it next to GASPI_Ext.h and uses nothing else from it.
#include "GASPI_Ext.h"
