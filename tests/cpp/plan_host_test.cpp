// Host-only checks of the C++ Plan layer (no GPU work: select / sku / can_implement /
// workspace_size are pure host functions, and an empty problem returns before any launch).
#include <cstdio>
#include <unordered_map>

#include "baracuda_kernels_q_plan.hpp"

using namespace baracuda;

static int failures = 0;
#define CHECK(cond)                                                          \
    do {                                                                     \
        if (!(cond)) {                                                       \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);    \
            ++failures;                                                      \
        }                                                                    \
    } while (0)

int main() {
    PlanPreference pref;
    W8A8GemmPlan p, raw;
    QGemmDescriptor desc{128, 1024, 1024, LayoutSku::Rcr, EpilogueKind::Identity};
    CHECK(W8A8GemmPlan::select(desc, pref, false, &p) == Error::Ok);
    CHECK(W8A8GemmPlan::select(desc, pref, true, &raw) == Error::Ok);
    CHECK(p.sku().arch == ArchSku::Sm100a && p.sku().backend == BackendKind::Bespoke);
    CHECK(p.sku().element == ElementKind::S8 && *p.sku().aux_element == ElementKind::Bf16);
    CHECK(p.precision_guarantee().accumulator == ElementKind::I32 && p.precision_guarantee().deterministic);
    CHECK(!(p.sku() == raw.sku()));
    std::unordered_map<KernelSku, int> cache;  // sku() is an autotuner cache key
    cache[p.sku()] = 1;
    W8A8GemmPlan again;
    W8A8GemmPlan::select(desc, pref, false, &again);
    CHECK(cache.count(again.sku()) == 1 && cache.count(raw.sku()) == 0);
    CHECK(p.workspace_size() == 0);

    QGemmDescriptor rrr = desc;
    rrr.layout = LayoutSku::Rrr;
    CHECK(W8A8GemmPlan::select(rrr, pref, false, &p) == Error::Ok);
    CHECK(*p.sku().layout == LayoutSku::Rrr);
    IntGemmPlan q8;
    CHECK(IntGemmPlan::select(desc, pref, ElementKind::S8, &q8) == Error::Ok);
    CHECK(q8.sku().element == ElementKind::S8 && !q8.sku().aux_element);
    CHECK(IntGemmPlan::select(desc, pref, ElementKind::Bf16, &q8) == Error::Unsupported);
    CHECK(IntGemmPlan::select(rrr, pref, ElementKind::Fp8E4M3, &q8) == Error::Ok);
    Q8OutGemmArgs qa;
    qa.lda = 1024;
    qa.ldb = 1024;
    qa.ldd = 1024;
    CHECK(q8.run(nullptr, Workspace::none(), qa) == Error::BufferTooSmall);  // the typed layer refuses empty views
    {
        GatedMlpUpPlan gp;
        GatedMlpUpDescriptor gd;
        gd.m = 64;
        gd.f = 48;
        gd.k = 128;
        CHECK(GatedMlpUpPlan::select(gd, pref, &gp) == Error::Unsupported);  // F in blocks of 32
        gd.f = 64;
        gd.scale_mode = ScaleMode::PerTensor;
        CHECK(GatedMlpUpPlan::select(gd, pref, &gp) == Error::InvalidProblem);  // s8 takes scale vectors
        gd.scale_mode = ScaleMode::PerRowCol;
        CHECK(GatedMlpUpPlan::select(gd, pref, &gp) == Error::Ok);
        CHECK(gp.sku().op == OP_GATED_MLP_UP && *gp.sku().aux_element == ElementKind::Bf16);
        CHECK(gp.workspace_size() == 0);
        auto fk = [](uintptr_t addr) { return reinterpret_cast<void*>(addr); };
        GatedMlpUpArgs ga;
        ga.a = {fk(0x10000), size_t(64) * 128};
        ga.lda = 128;
        ga.b_gate_up = {fk(0x20000), size_t(128) * 128};
        ga.ldb = 128;
        ga.d = {fk(0x40000), size_t(64) * 64};
        ga.ldd = 64;
        ga.scale_a = {static_cast<const float*>(fk(0x60000)), 64};
        ga.scale_b = {static_cast<const float*>(fk(0x61000)), 64};
        CHECK(gp.can_implement(ga) == Error::BufferTooSmall);  // scale_b covers gate and up
        ga.scale_b.len = 128;
        CHECK(gp.can_implement(ga) == Error::Ok);
        ga.ldd = 60;
        CHECK(gp.can_implement(ga) == Error::InvalidProblem);
        ga.ldd = 68;
        CHECK(gp.can_implement(ga) == Error::MisalignedOperand);
    }
    QGemmDescriptor bias = desc;
    bias.epilogue = EpilogueKind::BiasRelu;
    CHECK(W8A8GemmPlan::select(bias, pref, true, &p) == Error::Unsupported);  // raw accumulators: identity only
    CHECK(W8A8GemmPlan::select(bias, pref, false, &p) == Error::Ok);
    CHECK(p.sku().epilogue && *p.sku().epilogue == EpilogueKind::BiasRelu);
    {
        auto fk = [](uintptr_t addr) { return reinterpret_cast<void*>(addr); };
        QGemmArgs y;
        y.a = {fk(0x10000), size_t(128) * 1024};
        y.lda = 1024;
        y.b = {fk(0x200000), size_t(1024) * 1024};
        y.ldb = 1024;
        y.d = {fk(0x400000), size_t(128) * 1024};
        y.ldd = 1024;
        y.scale_a = {static_cast<const float*>(fk(0x600000)), 128};
        y.scale_b = {static_cast<const float*>(fk(0x601000)), 1024};
        CHECK(p.can_implement(y) == Error::InvalidProblem);  // the chain needs a bias
        y.bias = {static_cast<const float*>(fk(0x602000)), 1000};
        CHECK(p.can_implement(y) == Error::BufferTooSmall);
        y.bias.len = 1024;
        CHECK(p.can_implement(y) == Error::Ok);
    }
    PlanPreference cublas;
    cublas.prefer_backend = BackendKind::Cublas;
    CHECK(W8A8GemmPlan::select(desc, cublas, false, &p) == Error::Unsupported);
    QGemmDescriptor neg = desc;
    neg.m = -1;
    CHECK(W8A8GemmPlan::select(neg, pref, false, &p) == Error::InvalidProblem);

    CHECK(W8A8GemmPlan::select(desc, pref, false, &p) == Error::Ok);
    auto fake = [](uintptr_t addr) { return reinterpret_cast<void*>(addr); };
    QGemmArgs x;
    x.a = {fake(0x10000), 128u * 1024u};
    x.lda = 1024;
    x.b = {fake(0x200000), 1024u * 1024u};
    x.ldb = 1024;
    x.d = {fake(0x400000), 128u * 1024u};
    x.ldd = 1024;
    x.scale_a = {static_cast<const float*>(fake(0x500000)), 128};
    x.scale_b = {static_cast<const float*>(fake(0x600000)), 1024};
    CHECK(p.can_implement(x) == Error::Ok);
    QGemmArgs y = x;
    y.b.len -= 1;
    CHECK(p.can_implement(y) == Error::BufferTooSmall);
    y = x;
    y.lda = 1000;
    CHECK(p.can_implement(y) == Error::InvalidProblem);
    y = x;
    y.lda = 1032;
    y.a.len = 128u * 1032u;
    CHECK(p.can_implement(y) == Error::MisalignedOperand);
    y = x;
    y.scale_b.len = 1023;
    CHECK(p.can_implement(y) == Error::BufferTooSmall);

    Fp8ScaledGemmPlan f;
    CHECK(Fp8ScaledGemmPlan::select(desc, pref, ScaleMode::PerTensor, false, &f) == Error::Ok);
    CHECK(f.sku().element == ElementKind::Fp8E4M3 && f.precision_guarantee().accumulator == ElementKind::F32);
    y = x;
    y.scale_a.len = 1;
    y.scale_b.len = 1;
    CHECK(f.can_implement(y) == Error::Ok);  // per-tensor scales are single floats

    GemvQ8Plan g;
    GemvQ8Descriptor gd{1, 14336, 4096, 1, LayoutSku::Rcr};
    CHECK(GemvQ8Plan::select(gd, pref, false, &g) == Error::Ok);
    CHECK(g.workspace_size() == 0);
    gd.layout = LayoutSku::Rrr;
    CHECK(GemvQ8Plan::select(gd, pref, false, &g) == Error::Ok);
    CHECK(g.workspace_size() > 0);
    PlanPreference tiny;
    tiny.max_workspace_bytes = 16;
    CHECK(GemvQ8Plan::select(gd, tiny, false, &g) == Error::Unsupported);
    gd.m = 9;
    CHECK(GemvQ8Plan::select(gd, pref, false, &g) == Error::InvalidProblem);

    // an empty problem runs to status 0 without touching the device
    W8A8GemmPlan e;
    CHECK(W8A8GemmPlan::select(QGemmDescriptor{0, 16, 16}, pref, false, &e) == Error::Ok);
    QGemmArgs ex;
    ex.lda = 16;
    ex.ldb = 16;
    ex.ldd = 16;
    ex.scale_a = {static_cast<const float*>(fake(0x500000)), 0};
    ex.scale_b = {static_cast<const float*>(fake(0x600000)), 16};
    CHECK(e.run(nullptr, Workspace::none(), ex) == Error::Ok);

    // the quantiser, the W8A8 linear built from it, and the SmoothQuant linear: selection rules and typed checks
    {
        QuantizePerTokenPlan qp;
        QuantizePerTokenDescriptor qd;
        qd.rows = 4;
        qd.cols = 4096;
        CHECK(QuantizePerTokenPlan::select(qd, pref, &qp) == Error::Ok);
        qd.q_max = 0;
        CHECK(QuantizePerTokenPlan::select(qd, pref, &qp) == Error::InvalidProblem);
        qd.q_max = 127;
        qd.input = ElementKind::S8;
        CHECK(QuantizePerTokenPlan::select(qd, pref, &qp) == Error::Unsupported);

        QuantizedLinearPlan ql;
        QuantizedLinearDescriptor ld;
        ld.m = 1;
        ld.c_out = 14336;
        ld.k = 4096;
        CHECK(QuantizedLinearPlan::select(ld, pref, &ql) == Error::Ok);
        CHECK(ql.sku().op == OP_GEMV_Q8 && *ql.sku().layout == LayoutSku::Rcr);  // decode: the streaming GEMV
        QuantizedLinearArgs la;
        la.activation = {fake(0x10000), 4096};
        la.weight_q = {static_cast<const int8_t*>(fake(0x100000)), size_t(14336) * 4096};
        la.weight_scale = {static_cast<const float*>(fake(0x8000000)), 14336};
        la.output = {fake(0x9000000), 14336};
        la.act_scale_scratch = {static_cast<float*>(fake(0x9100000)), 1};
        CHECK(ql.fused_decode(la));  // bf16 activations, m <= 8, K = 8 x 512: one launch
        la.activation.ptr = fake(0x10008);
        CHECK(!ql.fused_decode(la));  // misaligned activations take the two-launch path
        la.activation.ptr = fake(0x10000);
        la.weight_scale.len = 14335;
        CHECK(ql.run(nullptr, Workspace::none(), la) == Error::BufferTooSmall);
        ld.m = 512;
        CHECK(QuantizedLinearPlan::select(ld, pref, &ql) == Error::Ok);
        CHECK(ql.sku().op == OP_W8A8_GEMM && !ql.fused_decode(la));  // prefill: the tcgen05 GEMM
        ld.activation_element = ElementKind::S8;
        CHECK(QuantizedLinearPlan::select(ld, pref, &ql) == Error::Unsupported);

        SmoothQuantLinearPlan sq;
        SmoothQuantLinearDescriptor sd;
        sd.m = 128;
        sd.n = 1024;
        sd.k = 1024;
        sd.act_scale = 0.02f;
        CHECK(SmoothQuantLinearPlan::select(sd, pref, &sq) == Error::Ok);
        CHECK(sq.sku().op == OP_SMOOTHQUANT_LINEAR && sq.workspace_size() == 0);
        SmoothQuantLinearArgs sa;
        sa.act_q = {static_cast<const int8_t*>(fake(0x10000)), size_t(128) * 1024};
        sa.weight_q = {static_cast<const int8_t*>(fake(0x200000)), size_t(1024) * 1024};
        sa.weight_scale = {static_cast<const float*>(fake(0x600000)), 1024};
        sa.output = {fake(0x400000), size_t(128) * 1024};
        CHECK(sq.can_implement(sa) == Error::Ok);
        sa.weight_scale.len = 1023;
        CHECK(sq.can_implement(sa) == Error::BufferTooSmall);
        sd.act_scale = 1.0f / 0.0f;
        CHECK(SmoothQuantLinearPlan::select(sd, pref, &sq) == Error::InvalidProblem);  // the scale must be finite
    }
    // dependent launches exist for the bf16-out plans only
    {
        W8A8GemmPlan r;
        CHECK(W8A8GemmPlan::select(desc, pref, true, &r) == Error::Ok);
        CHECK(r.run_dependent(nullptr, Workspace::none(), x) == Error::Unsupported);
        W8A8GemmPlan e2;
        CHECK(W8A8GemmPlan::select(QGemmDescriptor{0, 16, 16}, pref, false, &e2) == Error::Ok);
        CHECK(e2.run_dependent(nullptr, Workspace::none(), ex) == Error::Ok);  // empty problem: status 0 before any launch
    }

    // tensor-parallel plans: sharding rules and the typed checks in front of the sharded C entry points
    {
        TensorParallelContext ctx{1, 4, nullptr};
        int32_t lo = 0, hi = 0;
        CHECK(shard_range(28672, ctx, &lo, &hi) == Error::Ok && lo == 7168 && hi == 14336);
        CHECK(shard_range(10, ctx, &lo, &hi) == Error::InvalidProblem);  // must divide evenly
        TensorParallelContext bad{4, 4, nullptr};
        CHECK(shard_range(16, bad, &lo, &hi) == Error::InvalidProblem);
        ColumnParallelQGemmPlan cp;
        CHECK(ColumnParallelQGemmPlan::make(ctx, 128, 1000, 512, ElementKind::S8, ScaleMode::PerRowCol, GatherMode::None,
                                            &cp) == Error::Ok);
        CHECK(cp.n_local() == 250 && cp.first_column() == 250);
        CHECK(ColumnParallelQGemmPlan::make(ctx, 128, 1001, 512, ElementKind::S8, ScaleMode::PerRowCol, GatherMode::None,
                                            &cp) == Error::InvalidProblem);
        CHECK(ColumnParallelQGemmPlan::make(ctx, 128, 1000, 512, ElementKind::Bf16, ScaleMode::PerRowCol, GatherMode::None,
                                            &cp) == Error::Unsupported);
        ColumnParallelArgs ca;
        CHECK(cp.forward(nullptr, ca) == Error::BufferTooSmall);  // empty views are refused before any launch
        ColumnParallelQGemmPlan cr;  // row-major [K, N] weight: the shard is a column range with the full row pitch
        CHECK(ColumnParallelQGemmPlan::make(ctx, 128, 1024, 512, ElementKind::S8, ScaleMode::PerRowCol,
                                            GatherMode::FusedMulticast, &cr, LayoutSku::Rrr) == Error::Ok);
        ca.a = {fake(0x10000), size_t(128) * 512};
        ca.w_local = {fake(0x200000), size_t(511) * 1024 + 256 - 1};
        ca.y_local = {fake(0x400000), size_t(128) * 256};
        CHECK(cr.forward(nullptr, ca) == Error::BufferTooSmall);  // one element short of (K - 1) * N + N / world
        ca.w_local.len += 1;
        CHECK(cr.forward(nullptr, ca) == Error::InvalidProblem);  // fused gather without the peer buffers
        RowParallelQGemmPlan rp;
        CHECK(RowParallelQGemmPlan::make(ctx, 64, 256, 4096, ElementKind::Fp8E4M3, ScaleMode::PerRowCol, ReduceMode::Nccl,
                                         &rp) == Error::Ok);
        CHECK(rp.k_local() == 1024 && rp.first_k() == 1024 && rp.workspace_size() == size_t(64) * 256 * 4);
        CHECK(RowParallelQGemmPlan::make(ctx, 64, 256, 4098, ElementKind::Fp8E4M3, ScaleMode::PerRowCol, ReduceMode::Nccl,
                                         &rp) == Error::InvalidProblem);
        RowParallelArgs ra;
        CHECK(rp.forward(nullptr, Workspace::none(), ra) == Error::WorkspaceTooSmall);
        void* fake_ptrs[4] = {fake(0x10000), fake(0x20000), fake(0x30000), fake(0x40000)};
        CHECK(rp.forward_fused(nullptr, ra, fake_ptrs, fake_ptrs, nullptr, nullptr) == Error::InvalidProblem);  // no way to meet
        CHECK(rp.forward_fused(nullptr, ra, fake_ptrs, fake_ptrs, fake_ptrs) == Error::BufferTooSmall);  // empty operand views
        CHECK(baracuda_q_peer_barrier_flag_bytes() == 128);
    }

    if (failures == 0) std::printf("plan_host_test ok\n");
    return failures == 0 ? 0 : 1;
}
