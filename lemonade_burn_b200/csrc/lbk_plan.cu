// Plans: a recorded decode-like sequence of fused ternary-linear groups replayed as one
// unit. Stands in for the reference's per-token loop of 120 parallel regions
// (crates/lb-ternary/benches/kbench.rs:148-194, crates/lb-model/src/model.rs:331-366).
#include <cstdlib>
#include <new>
#include <vector>

#include "lbk_internal.cuh"

namespace lbk {

struct Plan {
    Ctx *ctx = nullptr;
    std::vector<GroupArgs> groups;
    // groups added without buffers get slots in plan-owned arenas (x then y, in add order)
    std::vector<int> arena_group;  // indices of such groups
    float *x_arena = nullptr, *y_arena = nullptr;
    size_t x_elems = 0, y_elems = 0;
    size_t weight_bytes = 0;
    bool finalized = false;
    // one persistent launch when every activation row fits a warp's slice of shared memory,
    // else a CUDA graph of one fused launch per group
    SweepTables *sweep = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    // lbk_plan_run_host pipelines the sweep against its own copies: the groups are cut into a few
    // segments of about equal weight bytes, each with its own sweep tables; segment s computes while
    // segment s+1's inputs come in and segment s-1's outputs go out (copy engines of both
    // directions and the SMs all busy). Streams and events are created once, here.
    struct Segment {
        SweepTables *sweep = nullptr;
        size_t x_off = 0, x_len = 0, y_off = 0, y_len = 0;  // in floats, inside the arenas
        cudaEvent_t in_done = nullptr, compute_done = nullptr;
    };
    std::vector<Segment> segments;
    cudaStream_t in_stream = nullptr, out_stream = nullptr;
    cudaEvent_t start = nullptr, out_done = nullptr;
};

static void plan_free_segments(Plan *p) {
    for (Plan::Segment &sg : p->segments) {
        if (sg.sweep) sweep_free(sg.sweep);
        if (sg.in_done) cudaEventDestroy(sg.in_done);
        if (sg.compute_done) cudaEventDestroy(sg.compute_done);
    }
    p->segments.clear();
    if (p->in_stream) cudaStreamDestroy(p->in_stream);
    if (p->out_stream) cudaStreamDestroy(p->out_stream);
    if (p->start) cudaEventDestroy(p->start);
    if (p->out_done) cudaEventDestroy(p->out_done);
    p->in_stream = p->out_stream = nullptr;
    p->start = p->out_done = nullptr;
}

// Cuts an all-arena plan into segments for the pipelined host path. Failure of any step just
// leaves the plan without segments (run_host then copies, runs and copies in sequence).
static void plan_build_segments(Plan *p) {
    const int want = 3;  // measured at the 2B4T sweep: 1 segment 198 us per step, 2: 180, 3: 174, 4: 184, 6: 210
    if (want < 2 || !p->sweep || p->arena_group.size() != p->groups.size() || p->groups.size() < static_cast<size_t>(2 * want)) return;
    size_t total = 0;
    for (const GroupArgs &g : p->groups)
        for (int i = 0; i < g.n; ++i) total += g.w[i]->rows * g.w[i]->rb;
    bool ok = cudaStreamCreateWithFlags(&p->in_stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p->out_stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&p->start, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&p->out_done, cudaEventDisableTiming) == cudaSuccess;
    size_t gi = 0, x_off = 0, y_off = 0, bytes_done = 0;
    for (int sidx = 0; sidx < want && ok; ++sidx) {
        Plan::Segment sg;
        sg.x_off = x_off;
        sg.y_off = y_off;
        std::vector<GroupArgs> sub;
        const size_t target = total * (sidx + 1) / want;
        while (gi < p->groups.size() && (bytes_done < target || sidx == want - 1)) {
            const GroupArgs &g = p->groups[gi++];
            sub.push_back(g);
            sg.x_len += g.w[0]->cols;
            for (int i = 0; i < g.n; ++i) {
                sg.y_len += g.w[i]->rows;
                bytes_done += g.w[i]->rows * g.w[i]->rb;
            }
        }
        x_off += sg.x_len;
        y_off += sg.y_len;
        ok = !sub.empty() && sweep_build(p->ctx, sub, &sg.sweep) == LBK_OK && sg.sweep != nullptr &&
             cudaEventCreateWithFlags(&sg.in_done, cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&sg.compute_done, cudaEventDisableTiming) == cudaSuccess;
        p->segments.push_back(sg);
    }
    if (!ok || gi != p->groups.size()) plan_free_segments(p);
}

int kernels_init(Ctx *ctx) {
    LBK_TRY(gemv_init(ctx));
    LBK_TRY(gemm_init(ctx));
    LBK_TRY(sweep_init(ctx));
    LBK_TRY(bf16_init(ctx));
    LBK_TRY(attn_tc_init(ctx));
    return LBK_OK;
}

}  // namespace lbk

using namespace lbk;

extern "C" {

int lbk_plan_create(lbk_ctx *c, lbk_plan **out) {
    if (!c || !out) return fail(LBK_ERR_INVALID, "lbk_plan_create: null argument");
    Plan *p = new (std::nothrow) Plan();
    if (!p) return fail(LBK_ERR_NOMEM, "out of host memory");
    p->ctx = reinterpret_cast<Ctx *>(c);
    *out = reinterpret_cast<lbk_plan *>(p);
    return LBK_OK;
}

int lbk_plan_add(lbk_plan *pl, const float *x_dev, const lbk_weight *const *ws, size_t n, float *const *outs_dev,
                 int32_t *const *iouts_dev) {
    if (!pl) return fail(LBK_ERR_INVALID, "plan is null");
    Plan *p = reinterpret_cast<Plan *>(pl);
    if (p->finalized) return fail(LBK_ERR_INVALID, "plan is already finalized");
    if (!ws || n < 1 || n > LBK_MAX_GROUP) return fail(LBK_ERR_INVALID, "group of %zu matrices (1..%d allowed)", n, LBK_MAX_GROUP);
    const bool arena = !x_dev && !outs_dev;
    if (!arena && (!x_dev || !outs_dev)) return fail(LBK_ERR_INVALID, "lbk_plan_add: give both x_dev and outs_dev, or neither");
    GroupArgs g;
    g.n = static_cast<int>(n);
    g.m = 1;
    g.x = x_dev;
    for (size_t i = 0; i < n; ++i) {
        const Weight *w = reinterpret_cast<const Weight *>(ws[i]);
        if (!w || w->ctx != p->ctx) return fail(LBK_ERR_INVALID, "matrix %zu is null or belongs to another context", i);
        if (w->cols != reinterpret_cast<const Weight *>(ws[0])->cols) return fail(LBK_ERR_SHAPE, "inner dimension mismatch in group");
        if (w->cols == 0 || w->rows == 0) return fail(LBK_ERR_UNSUPPORTED, "plans take non-empty matrices");
        if (!arena && !outs_dev[i]) return fail(LBK_ERR_INVALID, "output %zu is null", i);
        g.w[i] = w;
        g.out[i] = arena ? nullptr : outs_dev[i];
        g.iout[i] = iouts_dev ? iouts_dev[i] : nullptr;
        p->weight_bytes += w->rows * w->rb;
    }
    if (!gemv_fits(p->ctx, g.w[0]->kp, 1)) return fail(LBK_ERR_UNSUPPORTED, "%zu columns do not fit the decode kernel", g.w[0]->cols);
    if (arena) {
        p->arena_group.push_back(static_cast<int>(p->groups.size()));
        p->x_elems += g.w[0]->cols;
        for (int i = 0; i < g.n; ++i) p->y_elems += g.w[i]->rows;
    }
    p->groups.push_back(g);
    return LBK_OK;
}

int lbk_plan_finalize(lbk_plan *pl) {
    if (!pl) return fail(LBK_ERR_INVALID, "plan is null");
    Plan *p = reinterpret_cast<Plan *>(pl);
    if (p->finalized) return LBK_OK;
    Ctx *ctx = p->ctx;
    LBK_CUDA(cudaSetDevice(ctx->device));
    if (!p->arena_group.empty()) {
        cudaError_t e = cudaMalloc(&p->x_arena, (p->x_elems + 4) * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc(&p->y_arena, (p->y_elems + 4) * sizeof(float));
        if (e != cudaSuccess) return fail(LBK_ERR_NOMEM, "plan arenas: %s", cudaGetErrorString(e));
        LBK_CUDA(cudaMemset(p->x_arena, 0, (p->x_elems + 4) * sizeof(float)));
        LBK_CUDA(cudaMemset(p->y_arena, 0, (p->y_elems + 4) * sizeof(float)));
        size_t xo = 0, yo = 0;
        for (int gi : p->arena_group) {
            GroupArgs &g = p->groups[gi];
            g.x = p->x_arena + xo;  // cols are multiples of 4 for every 16-byte aligned slot
            xo += g.w[0]->cols;
            for (int i = 0; i < g.n; ++i) {
                g.out[i] = p->y_arena + yo;
                yo += g.w[i]->rows;
            }
        }
    }
    if (!p->groups.empty()) {
        int st_sweep = sweep_build(ctx, p->groups, &p->sweep);
        if (st_sweep != LBK_OK && st_sweep != LBK_ERR_UNSUPPORTED) return st_sweep;
    }
    if (!p->groups.empty() && !p->sweep) {
        cudaStream_t st = ctx->own_stream;
        LBK_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        int status = LBK_OK;
        const uint64_t before = ctx->launches;
        for (const GroupArgs &g : p->groups) {
            status = launch_gemv(ctx, g, st);
            if (status != LBK_OK) break;
        }
        ctx->launches = before;  // recording is not launching
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamEndCapture(st, &graph);
        if (status != LBK_OK) {
            if (graph) cudaGraphDestroy(graph);
            return status;
        }
        if (e != cudaSuccess) return fail(LBK_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        p->graph = graph;
        LBK_CUDA(cudaGraphInstantiate(&p->exec, graph, 0));
    }
    plan_build_segments(p);
    p->finalized = true;
    return LBK_OK;
}

int lbk_plan_run(lbk_plan *pl, void *stream) {
    if (!pl) return fail(LBK_ERR_INVALID, "plan is null");
    Plan *p = reinterpret_cast<Plan *>(pl);
    if (!p->finalized) return fail(LBK_ERR_INVALID, "plan is not finalized");
    LBK_CUDA(cudaSetDevice(p->ctx->device));
    if (p->sweep) return sweep_launch(p->ctx, p->sweep, static_cast<cudaStream_t>(stream));
    if (!p->exec) return LBK_OK;
    LBK_CUDA(cudaGraphLaunch(p->exec, static_cast<cudaStream_t>(stream)));
    p->ctx->launches += p->groups.size();
    return LBK_OK;
}

int lbk_plan_run_host(lbk_plan *pl, const float *x_host, size_t x_len, float *y_host, size_t y_len, void *stream) {
    if (!pl) return fail(LBK_ERR_INVALID, "plan is null");
    Plan *p = reinterpret_cast<Plan *>(pl);
    if (!p->finalized) return fail(LBK_ERR_INVALID, "plan is not finalized");
    if (p->arena_group.size() != p->groups.size())
        return fail(LBK_ERR_INVALID, "lbk_plan_run_host needs every group added without device buffers");
    if (x_len != p->x_elems || y_len != p->y_elems)
        return fail(LBK_ERR_SHAPE, "host arenas: got %zu inputs / %zu outputs, plan has %zu / %zu", x_len, y_len, p->x_elems, p->y_elems);
    if ((x_len && !x_host) || (y_len && !y_host)) return fail(LBK_ERR_INVALID, "host buffer is null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LBK_CUDA(cudaSetDevice(p->ctx->device));
    if (!p->segments.empty()) {
        // inputs of every segment queue up on the inbound stream; a segment's sweep waits for its own
        // inputs only, and its outputs leave on the outbound stream while the next segment computes
        LBK_CUDA(cudaEventRecord(p->start, st));
        LBK_CUDA(cudaStreamWaitEvent(p->in_stream, p->start, 0));
        LBK_CUDA(cudaStreamWaitEvent(p->out_stream, p->start, 0));
        for (Plan::Segment &sg : p->segments) {
            LBK_CUDA(cudaMemcpyAsync(p->x_arena + sg.x_off, x_host + sg.x_off, sg.x_len * sizeof(float), cudaMemcpyHostToDevice, p->in_stream));
            LBK_CUDA(cudaEventRecord(sg.in_done, p->in_stream));
        }
        for (Plan::Segment &sg : p->segments) {
            LBK_CUDA(cudaStreamWaitEvent(st, sg.in_done, 0));
            LBK_TRY(sweep_launch(p->ctx, sg.sweep, st));
            LBK_CUDA(cudaEventRecord(sg.compute_done, st));
            LBK_CUDA(cudaStreamWaitEvent(p->out_stream, sg.compute_done, 0));
            LBK_CUDA(cudaMemcpyAsync(y_host + sg.y_off, p->y_arena + sg.y_off, sg.y_len * sizeof(float), cudaMemcpyDeviceToHost, p->out_stream));
        }
        LBK_CUDA(cudaEventRecord(p->out_done, p->out_stream));
        LBK_CUDA(cudaStreamWaitEvent(st, p->out_done, 0));
        LBK_CUDA(cudaStreamSynchronize(st));
        return LBK_OK;
    }
    if (x_len) LBK_CUDA(cudaMemcpyAsync(p->x_arena, x_host, x_len * sizeof(float), cudaMemcpyHostToDevice, st));
    LBK_TRY(lbk_plan_run(pl, stream));
    if (y_len) LBK_CUDA(cudaMemcpyAsync(y_host, p->y_arena, y_len * sizeof(float), cudaMemcpyDeviceToHost, st));
    LBK_CUDA(cudaStreamSynchronize(st));
    return LBK_OK;
}

size_t lbk_plan_input_elems(const lbk_plan *pl) { return pl ? reinterpret_cast<const Plan *>(pl)->x_elems : 0; }
size_t lbk_plan_output_elems(const lbk_plan *pl) { return pl ? reinterpret_cast<const Plan *>(pl)->y_elems : 0; }
const float *lbk_plan_input_arena(const lbk_plan *pl) { return pl ? reinterpret_cast<const Plan *>(pl)->x_arena : nullptr; }
const float *lbk_plan_output_arena(const lbk_plan *pl) { return pl ? reinterpret_cast<const Plan *>(pl)->y_arena : nullptr; }

size_t lbk_plan_weight_bytes(const lbk_plan *pl) { return pl ? reinterpret_cast<const Plan *>(pl)->weight_bytes : 0; }

int lbk_plan_destroy(lbk_plan *pl) {
    if (!pl) return LBK_OK;
    Plan *p = reinterpret_cast<Plan *>(pl);
    if (p->sweep) sweep_free(p->sweep);
    plan_free_segments(p);
    if (p->exec) cudaGraphExecDestroy(p->exec);
    if (p->graph) cudaGraphDestroy(p->graph);
    if (p->x_arena) cudaFree(p->x_arena);
    if (p->y_arena) cudaFree(p->y_arena);
    delete p;
    return LBK_OK;
}

}  // extern "C"
