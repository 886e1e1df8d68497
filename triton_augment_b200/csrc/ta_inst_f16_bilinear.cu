#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f16_bilinear() { return make_table<__half, 2>(); }
}
