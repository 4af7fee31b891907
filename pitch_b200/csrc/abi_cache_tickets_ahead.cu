// cache_decode_kernel<..., 2>: items dealt by drawn tickets, the items ahead asked of the L2 (short launches).
#define PITCH_TICKET_DEAL 2
#include "abi_cache_tickets_impl.h"
