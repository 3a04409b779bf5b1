"""Run the reference's own CUDA library (oracle/_ref/libcudaBERT_ref.so, built by
oracle/build_ref.py) on one batch and save its pooler output.  TEST INFRASTRUCTURE.

    python oracle/run_ref_cuda.py <weight_dir> <large 0|1> <inputs.npz> <out.npy> [timed calls]

With `timed calls` it repeats the call that many times after two warm-up calls and prints one JSON
line with the wall-clock rate (Cuda_Bert returns after its device-to-host copy).

Runs in a process of its own: the reference exits the process on any error
(cuda_bert/utils/common.h:58-65) and exports the same symbol names as the product library.
`inputs.npz` holds int32 ids, seg and (optionally) mask of shape [B, S].  Calls, unmodified, the
reference's init_model / Cuda_Bert / release_model (cuda_bert/cuda_bert.cu:26-70)."""
import ctypes
import json
import os
import sys
import time

import numpy as np
from numpy.ctypeslib import ndpointer


def main():
    wdir, large, inp, out = sys.argv[1], bool(int(sys.argv[2])), sys.argv[3], sys.argv[4]
    here = os.path.dirname(os.path.abspath(__file__))
    lib = ctypes.CDLL(os.path.join(here, "_ref", "libcudaBERT_ref.so"))
    lib.init_model.argtypes = [ctypes.c_bool, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_char_p]
    lib.init_model.restype = ctypes.c_void_p
    lib.release_model.argtypes = [ctypes.c_void_p]
    i32 = ndpointer(np.int32, flags="C_CONTIGUOUS")
    lib.Cuda_Bert.argtypes = [ctypes.c_void_p, ndpointer(np.float32, flags="C_CONTIGUOUS"), i32, i32, ctypes.c_int,
                              ctypes.c_int, ctypes.c_void_p]
    data = np.load(inp)
    ids = np.ascontiguousarray(data["ids"], np.int32)
    seg = np.ascontiguousarray(data["seg"], np.int32)
    mask = np.ascontiguousarray(data["mask"], np.int32) if "mask" in data.files else None
    B, S = ids.shape
    model = lib.init_model(large, 0, B, S, wdir.encode())
    H = 1024 if large else 768
    res = np.zeros((B, H), np.float32)
    mptr = None if mask is None else mask.ctypes.data_as(ctypes.c_void_p)
    lib.Cuda_Bert(model, res, ids, seg, B, S, mptr)
    np.save(out, res)
    iters = int(sys.argv[5]) if len(sys.argv) > 5 else 0
    if iters > 0:
        lib.Cuda_Bert(model, res, ids, seg, B, S, mptr)
        t0 = time.perf_counter()
        for _ in range(iters):
            lib.Cuda_Bert(model, res, ids, seg, B, S, mptr)
        dt = time.perf_counter() - t0
        print(json.dumps({"sequences_per_s": B * iters / dt, "ms_per_batch": dt / iters * 1e3, "batch": B, "seq": S,
                          "calls": iters}), flush=True)
    lib.release_model(model)


if __name__ == "__main__":
    main()
