"""Every library the package can load, with the variants (compile-time sizes)
that are built ahead of time.  A library outside this list is still compiled
at its first use."""
from __future__ import annotations


def all_variants():
    """[(source, defines, extra flags)] for `compile_many`."""
    jobs = [
        ("elementwise.cu", (), ()),
        ("attention_generic.cu", (), ()),
        ("gemm_f32.cu", (), ()),
        ("sampling.cu", (), ()),
        ("linear_small_m.cu", (), ()),
        ("gemm_tcgen05.cu", (), ()),
        ("ffn_small_m.cu", (), ()),
        ("linear_stream.cu", (), ()),
        ("stream_probe.cu", (), ()),
        ("linear_ring.cu", (), ()),
    ]
    for head_dim in (16, 32, 48, 64, 128):
        jobs.append(("attention_decode.cu", (f"HEAD_DIM={head_dim}",), ()))
    for head_dim in (16, 32, 48, 64, 128):
        jobs.append(("attention_prefill.cu", (f"HEAD_DIM={head_dim}",), ()))
    for head_dim in (64, 128):
        jobs.append(("attention_tcgen05.cu", (f"HEAD_DIM={head_dim}",), ()))
    for head_dim in (64, 128):
        jobs.append(("layer_small_m.cu", (f"HEAD_DIM={head_dim}",), ()))
    return jobs
