// placeholder, replaced below
#include "uccl_net.h"
