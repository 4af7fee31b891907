// cache_decode_kernel<..., 1>: items dealt by drawn tickets.
#define PITCH_TICKET_DEAL 1
#include "abi_cache_tickets_impl.h"
