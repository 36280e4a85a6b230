// Library-internal view of an AfirtRowsumExchange (include/CAPI/RuntimeCuda.h): what a launch needs from it.
#pragma once

#include "CAPI/RuntimeCuda.h"
#include "common/status.h"
#include "kernels/kernels.h"

namespace afir {

// Fills `record` for the exchange's NEXT call (call number, mailbox half, peer addresses) and reports the device
// the mailbox lives on.  Nothing changes until commitExchangeCall() is called after a successful launch, so a
// launch that fails on the host leaves every rank's call numbers in step.
Status nextExchangeCall(AfirtRowsumExchange exchange, kernels::RowReduceExchange &record, int &device);
void commitExchangeCall(AfirtRowsumExchange exchange, const kernels::RowReduceExchange &record);

} // namespace afir
