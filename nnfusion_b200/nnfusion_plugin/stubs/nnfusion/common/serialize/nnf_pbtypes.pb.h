// Stand-in for the header protoc generates from src/nnfusion/common/serialize/nnf_pbtypes.proto, for syntax checks of
// the plugin sources where protoc is not installed: the enumeration the compiler's headers name, nothing else.
#pragma once
namespace nnfusion
{
    namespace serialize
    {
        enum PBType
        {
            DT_INVALID = 0,
            DT_BOOL = 1,
            DT_CHAR = 2,
            DT_FLOAT = 3,
            DT_DOUBLE = 4,
            DT_INT8 = 5,
            DT_INT16 = 6,
            DT_INT32 = 7,
            DT_INT64 = 8,
            DT_UINT8 = 9,
            DT_UINT16 = 10,
            DT_UINT32 = 11,
            DT_UINT64 = 12
        };
    }
}
