"""Times every fp32 kernel variant of the library on a grid of shapes, beside the automatic choice and
cuBLAS (`torch.matmul`, TF32 off): the measurement behind the automatic choice in `vt_sgemm`.

    python -m veritac_b200.shape_sweep            # the built-in grid
    python -m veritac_b200.shape_sweep 8192x16x8192 300x8192x8192

Device-resident operands, CUDA events on the launching stream, 10 launches after 2 warm-up launches per
cell.  Needs a GPU; there is no CPU path.
"""
from __future__ import annotations

import sys

GRID = ((256, 256, 256), (512, 512, 512), (768, 768, 768), (1024, 1024, 1024), (2048, 2048, 2048), (256, 256, 8192),
        (512, 512, 8192), (1024, 256, 4096), (8192, 16, 8192), (8192, 64, 8192), (8192, 128, 8192), (8192, 256, 8192),
        (65536, 16, 1024), (4096, 32, 4096), (2048, 64, 2048), (16384, 128, 512), (16, 8192, 8192), (64, 8192, 8192),
        (128, 8192, 8192), (300, 8192, 8192), (384, 4096, 4096), (512, 8192, 8192), (1024, 8192, 1024), (128, 512, 512),
        (200, 300, 400), (2000, 200, 2000), (4096, 4096, 256), (4096, 4096, 64), (8192, 8192, 128), (128, 128, 65536),
        (1024, 64, 16384), (640, 640, 640), (1536, 1536, 1536), (3072, 512, 3072), (512, 3072, 3072))


def main(argv) -> int:
    import torch

    from . import _native as nv

    torch.backends.cuda.matmul.allow_tf32 = False
    shapes = [tuple(int(x) for x in a.lower().split("x")) for a in argv] or list(GRID)
    names = {nv.VT_SGEMM_TILE128: "tile128", nv.VT_SGEMM_TILE64: "tile64", nv.VT_SGEMM_TILE32: "tile32",
             nv.VT_SGEMM_TF32X3: "tf32x3", nv.VT_SGEMM_PANEL_TF32X3: "panel", nv.VT_SGEMM_TALL_TF32X3: "tall"}
    st = nv.torch_stream()

    def timed(fn) -> float:
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 10

    print("| M x N x K | automatic | best single variant | automatic / best | cuBLAS | automatic / cuBLAS | "
          + " | ".join(names.values()) + " |")
    print("|---|---|---|---|---|---|" + "---|" * len(names))
    for (m, n, k) in shapes:
        A = torch.rand((m, k), device="cuda") * 2 - 1
        B = torch.rand((k, n), device="cuda") * 2 - 1
        C = torch.empty((m, n), device="cuda")
        cells = {}
        for variant in names:
            if variant == nv.VT_SGEMM_PANEL_TF32X3 and m > 512:
                continue
            try:
                cells[variant] = timed(lambda: nv.sgemm(A, B, C, m, n, k, variant=variant, where=nv.VT_DEVICE, stream=st))
                nv.sync(0, st)
            except nv.NativeError:
                pass
        auto = timed(lambda: nv.sgemm(A, B, C, m, n, k, where=nv.VT_DEVICE, stream=st))
        nv.sync(0, st)
        lib = timed(lambda: torch.matmul(A, B, out=C))
        best = min(cells, key=cells.get)
        print("| %d x %d x %d | %.4f ms | %s %.4f | %.2f | %.4f | %.2f | " % (m, n, k, auto, names[best], cells[best],
                                                                        auto / cells[best], lib, auto / lib)
              + " | ".join("%.4f" % cells[v] if v in cells else "-" for v in names) + " |", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
