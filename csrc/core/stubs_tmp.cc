#include "enqueue.h"
#include "../rma/rma.h"
namespace uccl {
ucclResult_t enqueueRing(Comm* c, const CollOp&, ucclProto_t, int) { commSetError(c, "ring: not built yet"); return ucclInvalidUsage; }
ucclResult_t enqueueCopyEngine(Comm* c, const CollOp&) { commSetError(c, "ce: not built yet"); return ucclInvalidUsage; }
void rmaDestroyAll(Comm*) {}
}
