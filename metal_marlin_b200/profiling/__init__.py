from .roofline import (KernelTimer, RooflinePoint, attention_flops, decode_step_cost, fp4_weight_bytes, fused_collective_roof_seconds,
                       gemm_flops, get_timer, load_peaks, profile_kernel, profile_records)
from .tracing import LaunchTracer, launch_tracer, record_event, trace_kernel, trace_scope, write_trace

__all__ = ["KernelTimer", "RooflinePoint", "attention_flops", "decode_step_cost", "fp4_weight_bytes", "fused_collective_roof_seconds",
           "gemm_flops", "get_timer", "load_peaks", "profile_kernel", "profile_records", "LaunchTracer", "launch_tracer", "record_event", "trace_kernel",
           "trace_scope", "write_trace"]
