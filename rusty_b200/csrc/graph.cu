// Stream capture / replay, device-side timing events and buffer fill.
#include "internal.h"

using namespace rusty;

extern "C" {

int rusty_cuda_graph_begin(rusty_cuda_ctx* ctx) {
    RUSTY_REQUIRE_CTX(ctx);
    if (ctx->capturing) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "graph_begin: a capture is already open");
    DeviceGuard g(ctx->device);
    int rc = check_cuda(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    if (rc) return rc;
    ctx->capturing = true;
    ctx->launches_at_capture = ctx->launches.load();
    return RUSTY_CUDA_OK;
}

int rusty_cuda_graph_end(rusty_cuda_ctx* ctx, rusty_cuda_graph** out) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!out) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "graph_end: null out pointer");
    *out = nullptr;
    if (!ctx->capturing) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "graph_end: no capture is open");
    DeviceGuard g(ctx->device);
    ctx->capturing = false;
    cudaGraph_t graph = nullptr;
    int rc = check_cuda(ctx, cudaStreamEndCapture(ctx->stream, &graph), "cudaStreamEndCapture");
    {   // releases that arrived while the capture was open
        std::vector<void*> ptrs;
        std::vector<rusty_cuda_graph*> graphs;
        {
            std::lock_guard<std::mutex> lk(ctx->pool_mu);
            ptrs.swap(ctx->deferred_free);
            graphs.swap(ctx->deferred_graphs);
        }
        if (!ptrs.empty() || !graphs.empty()) cudaStreamSynchronize(ctx->stream);
        for (void* p : ptrs) cudaFree(p);
        for (rusty_cuda_graph* g2 : graphs) {
            cudaGraphExecDestroy(g2->exec);
            cudaGraphDestroy(g2->graph);
            delete g2;
        }
    }
    if (rc) return rc;
    uint64_t recorded = ctx->launches.load() - ctx->launches_at_capture;
    // Captured launches did not run: take them back out of the counter; each
    // replay adds them.
    ctx->launches.store(ctx->launches_at_capture);
    cudaGraphExec_t exec = nullptr;
    rc = check_cuda(ctx, cudaGraphInstantiate(&exec, graph, 0), "cudaGraphInstantiate");
    if (rc) {
        cudaGraphDestroy(graph);
        return rc;
    }
    rusty_cuda_graph* gr = new (std::nothrow) rusty_cuda_graph();
    if (!gr) {
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(graph);
        return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "graph_end: host allocation failed");
    }
    gr->ctx = ctx;
    gr->graph = graph;
    gr->exec = exec;
    gr->kernels = recorded;
    *out = gr;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_graph_launch(rusty_cuda_ctx* ctx, rusty_cuda_graph* graph) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!graph || graph->ctx != ctx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "graph_launch: graph is null or foreign");
    if (ctx->capturing) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "graph_launch: a capture is open");
    DeviceGuard g(ctx->device);
    int rc = check_cuda(ctx, cudaGraphLaunch(graph->exec, ctx->stream), "cudaGraphLaunch");
    if (rc) return rc;
    count_launch(ctx, graph->kernels);
    return RUSTY_CUDA_OK;
}

int rusty_cuda_graph_destroy(rusty_cuda_graph* graph) {
    if (!graph) return RUSTY_CUDA_OK;
    if (graph->ctx->capturing) {   // destroyed while another capture is open on its context: after that capture
        std::lock_guard<std::mutex> lk(graph->ctx->pool_mu);
        graph->ctx->deferred_graphs.push_back(graph);
        return RUSTY_CUDA_OK;
    }
    DeviceGuard g(graph->ctx->device);
    cudaStreamSynchronize(graph->ctx->stream);
    cudaGraphExecDestroy(graph->exec);
    cudaGraphDestroy(graph->graph);
    delete graph;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_event_create(rusty_cuda_ctx* ctx, rusty_cuda_event** out) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!out) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "event_create: null out pointer");
    *out = nullptr;
    DeviceGuard g(ctx->device);
    cudaEvent_t e = nullptr;
    int rc = check_cuda(ctx, cudaEventCreate(&e), "cudaEventCreate");
    if (rc) return rc;
    rusty_cuda_event* ev = new (std::nothrow) rusty_cuda_event();
    if (!ev) {
        cudaEventDestroy(e);
        return fail(ctx, RUSTY_CUDA_ERR_MEMORY_ALLOCATION, "event_create: host allocation failed");
    }
    ev->ctx = ctx;
    ev->ev = e;
    *out = ev;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_event_record(rusty_cuda_ctx* ctx, rusty_cuda_event* ev) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!ev || ev->ctx != ctx) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "event_record: event is null or foreign");
    DeviceGuard g(ctx->device);
    return check_cuda(ctx, cudaEventRecord(ev->ev, ctx->stream), "cudaEventRecord");
}

int rusty_cuda_event_elapsed_ms(rusty_cuda_ctx* ctx, rusty_cuda_event* start, rusty_cuda_event* stop, float* ms) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!start || !stop || !ms) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "event_elapsed_ms: null argument");
    DeviceGuard g(ctx->device);
    int rc = check_cuda(ctx, cudaEventSynchronize(stop->ev), "cudaEventSynchronize");
    if (rc) return rc;
    return check_cuda(ctx, cudaEventElapsedTime(ms, start->ev, stop->ev), "cudaEventElapsedTime");
}

int rusty_cuda_event_destroy(rusty_cuda_event* ev) {
    if (!ev) return RUSTY_CUDA_OK;
    DeviceGuard g(ev->ctx->device);
    cudaEventDestroy(ev->ev);
    delete ev;
    return RUSTY_CUDA_OK;
}

int rusty_cuda_buf_fill_u8(rusty_cuda_ctx* ctx, rusty_cuda_buf* buf, size_t offset, int value, size_t bytes) {
    RUSTY_REQUIRE_CTX(ctx);
    if (!buf) return fail(ctx, RUSTY_CUDA_ERR_INVALID_OPERATION, "buf_fill: null buffer");
    if (offset > buf->bytes || bytes > buf->bytes - offset)
        return fail(ctx, RUSTY_CUDA_ERR_BUFFER_OPERATION, "buf_fill: range [%zu, %zu) exceeds the buffer's %zu bytes", offset,
                    offset + bytes, buf->bytes);
    if (bytes == 0) return RUSTY_CUDA_OK;
    DeviceGuard g(ctx->device);
    return check_cuda(ctx, cudaMemsetAsync((char*)buf->ptr + offset, value, bytes, ctx->stream), "cudaMemsetAsync");
}

}  // extern "C"
