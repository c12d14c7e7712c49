"""Time-breakdown tool on synthetic kernel timelines (classes, overlap rule, idle split)."""
import json

from multimesh_jax_b200.utils.timeline import Span, breakdown, classify, spans_from_chrome_trace


def test_kernel_classes():
    assert classify("ncclDevKernel_AllGather_RING_LL(ncclDevKernelArgsStorage<4096ul>)") == "NCCL AG"
    assert classify("ncclDevKernel_ReduceScatter_Sum_bf16_RING_LL") == "NCCL AR/RS"
    assert classify("ncclDevKernel_SendRecv(ncclDevKernelArgsStorage<4096ul>)") == "NCCL other"
    assert classify("void mm::reshard_pull_kernel<4>(mm::PullArgs)") == "Reshard"
    assert classify("void mm::gemm_bf16_kernel<false, false, mm::AllReduceHook>(...)") == "Fused comm"
    assert classify("void mm::gemm_bf16_kernel<false, false, mm::PlainHook<0> >(...)") == "Compute"
    assert classify("Memcpy DtoD (Device -> Device)") == "Memcpy"


def test_breakdown_charges_hidden_communication_to_compute_and_splits_idle():
    spans = [
        Span("mm.task:fwd0", 0, 100, 0, "range"),
        Span("gemm", 0, 40, 0), Span("ncclDevKernel_AllReduce_Sum", 30, 30, 0),   # 10 us hidden under the GEMM
        Span("rmsnorm", 70, 10, 0),
        Span("mm.task:bwd0", 200, 50, 0, "range"),
        Span("gemm", 200, 50, 0),
        Span("gemm", 0, 1000, 1),                                                  # another device: ignored
    ]
    b = breakdown(spans, device=0)
    assert b.wall_us == 250
    assert b.classes["Compute"] == 100
    assert b.classes["NCCL AR/RS"] == 20
    assert b.classes["CUDA idle"] == 30          # inside fwd0: 60..70 and 80..100
    assert b.classes["Pipeline idle"] == 100     # between the two tasks
    assert abs(sum(b.classes.values()) - b.wall_us) < 1e-6
    assert b.per_task["fwd0"]["count"] == 1 and b.top_kernels[0][0] == "gemm"
    assert "Pipeline idle" in b.format() and json.dumps(b.to_dict())


def test_chrome_trace_reader(tmp_path):
    doc = {"traceEvents": [
        {"ph": "X", "cat": "kernel", "name": "gemm", "ts": 10, "dur": 5, "args": {"device": 0}},
        {"ph": "X", "cat": "gpu_user_annotation", "name": "mm.task:t", "ts": 8, "dur": 10, "args": {"device": 0}},
        {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 0, "dur": 5},
        {"ph": "i", "name": "marker", "ts": 0}]}
    p = tmp_path / "trace.json"
    p.write_text(json.dumps(doc))
    spans = spans_from_chrome_trace(str(p))
    assert [(s.name, s.kind) for s in spans] == [("gemm", "kernel"), ("mm.task:t", "range")]


def test_event_edges_of_the_runtime_context_appear_in_the_breakdown():
    """A context that records cross-stream event edges (the fake-API form of the CUDA context
    here) hands them to the breakdown, which lists them by stream pair."""
    from multimesh_jax_b200 import _mm_C
    from multimesh_jax_b200.utils import timeline
    ctx = _mm_C.CudaContext([0], [0], [0], fake=True)
    ctx.open_window()
    ctx.create_execute_task(0, [], [(1, 0)], lambda: None, "produce", False, 0, 0, 0)      # compute stream writes buffer 1
    ctx.reshard(0, [(1, 0)], [(2, 0)], lambda: None, "reshard S1->S2", 0, 1)                # communication stream reads it
    ctx.create_execute_task(0, [(2, 0)], [(3, 0)], lambda: None, "consume", False, 0, 0, 0)
    ctx.close_window()
    b = timeline.Breakdown(0, 1000.0)
    b.event_edges = list(ctx.edges())
    summary = b.edge_summary()
    assert summary["compute->communication"]["count"] == 1
    assert summary["communication->compute"]["count"] == 1
    assert "produce -> reshard S1->S2" in summary["compute->communication"]["examples"][0]
    text = b.format()
    assert "event edges between streams: 2" in text
    assert b.to_dict()["event_edges"] == summary
    ctx.shutdown()
