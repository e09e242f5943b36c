#include "operators.h"

#if !defined(PSB_OPERATOR_PLUGIN)
// The registry of this process (see operator.h). Default visibility: plug-in libraries bind to it.
extern "C" __attribute__((visibility("default"))) void* psb_operator_factory() {
    static psb::OperatorFactory factory;
    return &factory;
}
#endif

namespace psb {

void register_builtin_operators() {
    static std::once_flag once;
    std::call_once(once, [] {
        auto& f = OperatorFactory::instance();
#define PSB_REG(cls) f.register_producer("psb", #cls, [](const Json& c) { return std::make_shared<cls>(c); })
        PSB_REG(SparseTableStorageOperator);
        PSB_REG(SparseTablePullOperator);
        PSB_REG(SparseTablePushOperator);
        PSB_REG(DirectPushOperator);
        PSB_REG(DenseTablePullOperator);
        PSB_REG(DenseTablePushOperator);
        PSB_REG(ForEachOperator);
        PSB_REG(ForEachWriteOperator);
        PSB_REG(EraseIfOperator);
        PSB_REG(DumpOperator);
        PSB_REG(LoadOperator);
        PSB_REG(RestoreOperator);
        PSB_REG(ShardUpdateContextOperator);
        PSB_REG(KVSyncOperator);
        PSB_REG(UDFOperator);
#undef PSB_REG
        // the dense storage operator is the sparse one with the dense partitioner
        f.register_producer("psb", "DenseTableStorageOperator", [](const Json& c) {
            Json d = c;
            d["partition"] = "dense";
            return std::make_shared<SparseTableStorageOperator>(d);
        });
    });
}

}  // namespace psb
