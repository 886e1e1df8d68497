#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f16_nearest() { return make_table<__half, 1>(); }
}
