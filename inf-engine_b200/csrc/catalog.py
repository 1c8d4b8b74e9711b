"""Which libraries exist and with which compile-time sizes they can be asked for."""

from __future__ import annotations

from .build import LIBRARIES


def all_build_requests():
    """(name, sources, defines, extra headers) of everything worth pre-building."""
    reqs = [("core", LIBRARIES["core"], {}, [])]
    reqs.append(("stream", ["gemm_stream.cu", "gemm_stream_tma.cu"], {}, []))
    reqs.append(("tcgen05", ["gemm_tcgen05.cu"], {}, []))
    reqs.append(("attn_tcgen05", ["attention_tcgen05.cu"], {}, []))
    for hd in (64, 128):
        reqs.append((f"attn_mma_hd{hd}", ["attention_mma.cu"], {"IE_HD": hd}, ["attention_noalloc.h"]))
    return reqs
