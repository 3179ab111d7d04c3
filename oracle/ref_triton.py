"""TEST INFRASTRUCTURE ONLY -- runs the reference's own Triton attention kernel on the GPU.

``oracle/build_ref.py --triton`` compiles ``_triton_mixed_sparse_attn_fwd_kernel`` of the reference
(ops/pit_sparse_flash_attention_v2.py:48-153) ahead of time into ``oracle/_ref``; this module loads
that binary through the CUDA driver API and launches it the way the reference's launcher does
(:156-192: grid ``(ceil(N/64), B*H)``, 128 threads, the argument order of the kernel signature).
The GPU parity tests compare the product kernel with its output.  Nothing here is used by the library.
"""
from __future__ import annotations

import ctypes
import json
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CUBIN = os.path.join(HERE, "_ref", "ref_triton_vs_fwd.cubin")

_CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8


def available() -> bool:
    return os.path.exists(CUBIN) and os.path.exists(CUBIN[:-6] + ".json")


class ReferenceTritonKernel:
    def __init__(self):
        self.meta = json.load(open(CUBIN[:-6] + ".json"))
        self.cu = ctypes.CDLL("libcuda.so.1")
        torch.zeros(1, device="cuda")                      # makes the primary context current on this thread
        image = open(CUBIN, "rb").read()
        self._image = ctypes.create_string_buffer(image, len(image))
        self.module = ctypes.c_void_p()
        self._ok(self.cu.cuModuleLoadData(ctypes.byref(self.module), self._image), "cuModuleLoadData")
        self.func = ctypes.c_void_p()
        self._ok(self.cu.cuModuleGetFunction(ctypes.byref(self.func), self.module, self.meta["name"].encode()), "cuModuleGetFunction")
        self._ok(self.cu.cuFuncSetAttribute(self.func, _CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                            int(self.meta["shared"])), "cuFuncSetAttribute")

    @staticmethod
    def _ok(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUDA driver error {rc}")

    def __call__(self, q, k, v, seqlens, block_count, block_offset, column_count, column_index, sm_scale):
        """Same tensors as ``_triton_mixed_sparse_attention`` (:156-168): ``q, k, v [B,H,N,128]`` bf16 with N a
        multiple of 64 and equal head counts, int32 index tensors in the reference format."""
        assert q.shape == k.shape == v.shape and q.shape[2] % 64 == 0 and q.shape[3] == 128 and q.dtype == torch.bfloat16
        o = torch.zeros_like(q)
        values = {
            "Q": q.data_ptr(), "K": k.data_ptr(), "V": v.data_ptr(), "seqlens": seqlens.data_ptr(), "sm_scale": float(sm_scale),
            "block_count": block_count.data_ptr(), "block_offset": block_offset.data_ptr(),
            "column_count": column_count.data_ptr(), "column_index": column_index.data_ptr(), "Out": o.data_ptr(),
            "Z": q.shape[0], "H": q.shape[1], "N_CTX": q.shape[2],
            "NUM_ROWS": block_count.shape[-1], "NNZ_S": block_offset.shape[-1], "NNZ_V": column_index.shape[-1],
        }
        for name, t in (("q", q), ("k", k), ("v", v), ("o", o)):
            for axis, st in zip(("z", "h", "m" if name in ("q", "o") else "n", "k"), t.stride()):
                values[f"stride_{name}{axis}"] = st
        holders = []
        for name, ty in self.meta["params"]:
            val = values[name]
            holders.append(ctypes.c_void_p(val) if ty.startswith("*") else ctypes.c_float(val) if ty == "fp32" else ctypes.c_int32(val))
        holders += [ctypes.c_void_p(0), ctypes.c_void_p(0)]       # global / profile scratch: sizes are 0 for this kernel
        argv = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.pointer(h), ctypes.c_void_p) for h in holders])
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._ok(self.cu.cuLaunchKernel(self.func, (q.shape[2] + 63) // 64, q.shape[0] * q.shape[1], 1,
                                        32 * int(self.meta["num_warps"]), 1, 1, int(self.meta["shared"]), stream, argv, None),
                 "cuLaunchKernel")
        return o


def reference_vertical_slash_attention(kernel: ReferenceTritonKernel, q, k, v, block_count, block_offset, column_count,
                                       column_index):
    """The reference's wrapper around the kernel (:206-242): zero-pad the sequence to a multiple of 64,
    repeat K/V to the query head count, ``sm_scale = d**-0.5``, slice the output back."""
    B, H, N, D = q.shape
    pad = (64 - N) & 63
    rep = H // k.shape[1]
    qp = torch.nn.functional.pad(q, [0, 0, 0, pad]).contiguous()
    kp = torch.nn.functional.pad(k.repeat_interleave(rep, 1), [0, 0, 0, pad]).contiguous()
    vp = torch.nn.functional.pad(v.repeat_interleave(rep, 1), [0, 0, 0, pad]).contiguous()
    seqlens = torch.tensor([N] * B, dtype=torch.int32, device=q.device)
    out = kernel(qp, kp, vp, seqlens, block_count, block_offset, column_count, column_index, D ** -0.5)
    return out[:, :, :N]
