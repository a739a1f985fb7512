"""Helpers for the GPU parity tests: torch is used only to hold device memory."""
import numpy as np
import torch

import primitiv_b200 as pb

MODES = {"3xtf32": pb.MODE_FP32_3XTF32, "tf32": pb.MODE_TF32, "fp16": pb.MODE_FP16,
         "3xfp16": pb.MODE_FP32_3XFP16}
# normwise relative error bounds against the fp64 oracle
TOL = {"3xtf32": 1e-5, "tf32": 2e-3, "fp16": 2e-3, "3xfp16": 1e-5}


def dev(x, mode):
    t = torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda()
    return t.half() if mode == pb.MODE_FP16 else t


def host(t):
    return t.float().cpu().numpy()


def matmul_fw(ctx, mode, a, b, di, dj, dk, ba, bb):
    da, db = dev(a, mode), dev(b, mode)
    y = torch.empty(di * dk * max(ba, bb), device="cuda", dtype=da.dtype)
    ctx.matmul_fw(mode, da.data_ptr(), db.data_ptr(), y.data_ptr(), di, dj, dk, ba, bb)
    torch.cuda.synchronize()
    assert ctx.status_poll() == 0
    return host(y)


def matmul_bw(ctx, mode, a, b, gy, ga0, gb0, di, dj, dk, ba, bb):
    da, db, dgy = dev(a, mode), dev(b, mode), dev(gy, mode)
    ga, gb = dev(ga0, mode), dev(gb0, mode)
    ctx.matmul_bw(mode, da.data_ptr(), db.data_ptr(), dgy.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                  di, dj, dk, ba, bb)
    torch.cuda.synchronize()
    assert ctx.status_poll() == 0
    return host(ga), host(gb)
