// Element-type codes shared by host launch code and kernels.
#pragma once
namespace uccl {
enum DevDataType : int { DEVDT_F16 = 0, DEVDT_BF16 = 1, DEVDT_F32 = 2 };
}
