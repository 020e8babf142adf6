/* <ODLA/odla.h> as HALO-generated model code includes it.  The declarations live in
 * ../odla_b200.h, which is binary compatible with the reference's ODLA/include/ODLA headers. */
#ifndef ODLA_B200_SHIM_ODLA_H_
#define ODLA_B200_SHIM_ODLA_H_
#include "../odla_b200.h"
#endif
