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
