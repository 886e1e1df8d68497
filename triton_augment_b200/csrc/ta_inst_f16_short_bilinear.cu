#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f16_short_bilinear() { return make_table<__half, 2, __half, kTileHShort>(); }
}
