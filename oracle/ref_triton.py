"""TEST INFRASTRUCTURE ONLY -- runs the reference's own Triton attention kernel on the GPU.

``oracle/build_ref.py --triton`` compiles ``_triton_mixed_sparse_attn_fwd_kernel``
(ops/pit_sparse_flash_attention_v2.py:48-153) and ``_triton_block_sparse_attn_fwd_kernel``
(ops/block_sparse_flash_attention.py:29-112) of the reference ahead of time into ``oracle/_ref``;
this module loads those binaries through the CUDA driver API and launches them the way the
reference's launchers do (grid ``(ceil(N/64), B*H)``, 128 threads, the argument order of the kernel
signature: v2 :156-192, block-sparse :115-148).  The streaming kernel's stage variants and the block-wise
prefill kernel of ``modules/flexprefill.py`` (:352-495) are built and launched the same way.
The GPU parity tests compare the product kernel with its output.  Nothing here is used by the library.
"""
from __future__ import annotations

import ctypes
import json
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CUBIN = os.path.join(HERE, "_ref", "ref_triton_vs_fwd.cubin")
CUBIN_BLOCK_SPARSE = os.path.join(HERE, "_ref", "ref_triton_bs_fwd.cubin")
CUBIN_128K_8HEADS = os.path.join(HERE, "_ref", "ref_triton_vs_fwd_128k_8heads.cubin")   # specialised like a JIT call
CUBIN_FLEX = os.path.join(HERE, "_ref", "ref_triton_flex_fwd.cubin")       # modules/flexprefill.py:352-495, 128-token blocks
CUBIN_FLEX_128K_8HEADS = os.path.join(HERE, "_ref", "ref_triton_flex_fwd_128k_8heads.cubin")   # specialised like a JIT call

_CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8


def available(cubin: str = CUBIN) -> bool:
    return os.path.exists(cubin) and os.path.exists(cubin[:-6] + ".json")


class ReferenceTritonKernel:
    def __init__(self, cubin: str = CUBIN):
        self.meta = json.load(open(cubin[:-6] + ".json"))
        self.cu = ctypes.CDLL("libcuda.so.1")
        torch.zeros(1, device="cuda")                      # makes the primary context current on this thread
        image = open(cubin, "rb").read()
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

    def launch(self, q, k, v, sm_scale, index_tensors: dict, sizes: dict):
        """``q, k, v [B,H,N,128]`` bf16, N a multiple of 64, equal head counts; ``index_tensors`` the int32
        pointer arguments by name, ``sizes`` the remaining integer arguments by name."""
        assert q.shape == k.shape == v.shape and q.shape[2] % 64 == 0 and q.shape[3] == 128 and q.dtype == torch.bfloat16
        o = torch.zeros_like(q)
        values = {"Q": q.data_ptr(), "K": k.data_ptr(), "V": v.data_ptr(), "Out": o.data_ptr(), "sm_scale": float(sm_scale),
                  "Z": q.shape[0], "H": q.shape[1], "N_CTX": q.shape[2]}
        values.update({name: t.data_ptr() for name, t in index_tensors.items()})
        values.update(sizes)
        for name, t in (("q", q), ("k", k), ("v", v), ("o", o)):
            for axis, st in zip(("z", "h", "m" if name in ("q", "o") else "n", "k"), t.stride()):
                values[f"stride_{name}{axis}"] = st
        self.launch_raw(values, ((q.shape[2] + 63) // 64, q.shape[0] * q.shape[1]))
        return o

    def launch_raw(self, values: dict, grid):
        """Launch with every kernel argument given by name (device addresses for pointers)."""
        for name, val in self.meta.get("example_ints", {}).items():       # a binary specialised for fixed sizes
            if values[name] != val:
                raise ValueError(f"this build of the kernel was specialised for {name}={val}, got {values[name]}")
        holders = []
        for name, ty in self.meta["params"]:
            val = values[name]
            holders.append(ctypes.c_void_p(val) if ty.startswith("*") else ctypes.c_float(val) if ty == "fp32" else ctypes.c_int32(val))
        holders += [ctypes.c_void_p(0), ctypes.c_void_p(0)]       # global / profile scratch: sizes are 0 for these kernels
        argv = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.pointer(h), ctypes.c_void_p) for h in holders])
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._ok(self.cu.cuLaunchKernel(self.func, int(grid[0]), int(grid[1]), int(grid[2]) if len(grid) > 2 else 1,
                                        32 * int(self.meta["num_warps"]), 1, 1,
                                        int(self.meta["shared"]), stream, argv, None), "cuLaunchKernel")

    def __call__(self, q, k, v, seqlens, block_count, block_offset, column_count, column_index, sm_scale):
        """Same tensors as ``_triton_mixed_sparse_attention`` (:156-168), index tensors in the reference format."""
        return self.launch(q, k, v, sm_scale,
                           {"seqlens": seqlens, "block_count": block_count, "block_offset": block_offset,
                            "column_count": column_count, "column_index": column_index},
                           {"NUM_ROWS": block_count.shape[-1], "NNZ_S": block_offset.shape[-1], "NNZ_V": column_index.shape[-1]})


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


def reference_block_sparse_attention(kernel: ReferenceTritonKernel, q, k, v, block_index):
    """The reference's ``block_sparse_attention`` around its kernel (ops/block_sparse_flash_attention.py:169-186):
    pad the sequence by ``64 - (N & 63)`` rows (a whole block when N is a multiple of 64, :178), repeat K/V to the
    query head count, ``sm_scale = d**-0.5``, slice back.  ``block_index [B,H,rows_pad,top_k]`` is given by the
    caller (sorted block ids; the kernel consumes the first ``min(m+1, top_k)`` of row m, :81)."""
    B, H, N, D = q.shape
    pad = 64 - (N & 63)
    rep = H // k.shape[1]
    qp = torch.nn.functional.pad(q, [0, 0, 0, pad]).contiguous()
    kp = torch.nn.functional.pad(k.repeat_interleave(rep, 1), [0, 0, 0, pad]).contiguous()
    vp = torch.nn.functional.pad(v.repeat_interleave(rep, 1), [0, 0, 0, pad]).contiguous()
    assert block_index.shape[2] == qp.shape[2] // 64
    seqlens = torch.tensor([N] * B, dtype=torch.int32, device=q.device)
    out = kernel.launch(qp, kp, vp, D ** -0.5, {"seqlens": seqlens, "block_index": block_index.contiguous()},
                        {"NUM_ROWS": block_index.shape[-2], "MAX_BLOCKS_PRE_ROW": block_index.shape[-1]})
    return out[:, :, :N]


def reference_flex_block_attention(kernel: ReferenceTritonKernel, q, k, v, block_mask, block_size: int = 128,
                                   softmax_scale: float | None = None, prepared_call: bool = False):
    """The reference's ``triton_block_wise_prefill_attention`` (modules/flexprefill.py:495-616) around its own kernel
    (:352-495): tensors in ``[B,N,H,D]`` layout, the block set as sorted flattened ids ``i*nb + j`` padded with
    ``nb*(nb+1)`` (:536-541), the per-row bins as counts + cumulative sum (the torch form of :312-350 given in the
    reference's comment), ``softmax_scale * log2(e)`` (:545-548), grid ``(B, H, nb)``.  ``q [B,H,N,128]``,
    ``k, v [B,Hkv,N,128]`` bf16 and ``block_mask [B,H,nb,nb]`` bool on the device; returns ``[B,H,N,128]``."""
    import math

    assert block_size == 128, "the binary was built for 128-token blocks"
    B, H, N, D = q.shape
    Hkv = k.shape[1]
    nb = (N + block_size - 1) // block_size
    qb, kb, vb = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    ob = torch.zeros_like(qb)
    lower = torch.tril(block_mask.to(torch.bool))
    counts = lower.sum(-1)                                                    # [B,H,nb]
    bins = torch.nn.functional.pad(torch.cumsum(counts, -1), (1, 0)).to(torch.int32).contiguous()
    width = int(counts.sum(-1).max().item())
    ids = torch.full((B, H, width), nb * (nb + 1), dtype=torch.int64, device=q.device)
    for b in range(B):
        for h in range(H):
            flat = lower[b, h].reshape(-1).nonzero().view(-1)               # row-major order = ascending ids
            ids[b, h, :flat.numel()] = flat
    scale = (1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale) * math.log2(math.e)
    values = {"q_ptr": qb.data_ptr(), "k_ptr": kb.data_ptr(), "v_ptr": vb.data_ptr(), "o_ptr": ob.data_ptr(),
              "block_idx_ptr": ids.data_ptr(), "idx_bin_ptr": bins.data_ptr(), "BATCH_SIZE": B, "NUM_HEADS": H,
              "NUM_KV_HEADS": Hkv, "GQA_GROUPS": H // Hkv, "Q_LEN": N, "K_LEN": N, "NUM_BLOCK": nb, "grid_offset": 0,
              "softmax_scale": scale}
    for name, t in (("q", qb), ("k", kb), ("v", vb), ("o", ob)):
        for axis, st in zip("bnhd", t.stride()):
            values[f"stride_{name}{axis}"] = st
    for axis, st in zip(("bb", "bh", "bt"), ids.stride()):
        values["stride_" + axis] = st
    for axis, st in zip(("ib", "ih", "it"), bins.stride()):
        values["stride_" + axis] = st
    launch = lambda: kernel.launch_raw(values, (B, H, nb))
    if prepared_call:
        # the launch alone (for timing) and the tensors it reads and writes, which must stay alive around it
        return launch, ob.transpose(1, 2), (qb, kb, vb, ids, bins)
    launch()
    torch.cuda.synchronize()
    return ob.transpose(1, 2)


def streaming_available() -> bool:
    return all(available(os.path.join(HERE, "_ref", f"ref_triton_stream_{stage}_{par}.cubin"))
               for stage in ("window", "sink", "single") for par in ("even", "ragged"))


def reference_streaming_forward(q, k, v, n_init: int, n_local: int):
    """The reference's ``streaming_forward`` (ops/streaming_kernel.py:611-646) with its own kernel ``_attn_fwd``:
    a window stage over all keys and, when the sequence is longer than the window, a second stage over the first
    ``n_init`` keys with the complement mask, fp32 O / M / L carried between the stages (:531-598, :420-499)."""
    B, H, N, D = q.shape
    assert n_init % 64 == 0, "only the compile-time variants with a sink count that is a multiple of 64 were built"
    rep = H // k.shape[1]
    q = q.contiguous()
    k = k.repeat_interleave(rep, 1).contiguous()          # the reference asserts q.shape == k.shape (:619)
    v = v.repeat_interleave(rep, 1).contiguous()
    round_len = (N + 63) // 64 * 64
    o = torch.empty((B, H, round_len, D), dtype=torch.float32, device=q.device)
    m = torch.empty((B, H, round_len), dtype=torch.float32, device=q.device)
    l = torch.empty((B, H, round_len), dtype=torch.float32, device=q.device)
    par = "even" if N % 64 == 0 else "ragged"

    def stage(tag, kk, vv):
        kern = ReferenceTritonKernel(os.path.join(HERE, "_ref", f"ref_triton_stream_{tag}_{par}.cubin"))
        values = {"Q": q.data_ptr(), "K": kk.data_ptr(), "V": vv.data_ptr(), "sm_scale": D ** -0.5,
                  "M": m.data_ptr(), "Out": o.data_ptr(), "L": l.data_ptr(),
                  "Z": B, "H": H, "H_KV": kk.shape[1], "N_CTX": N, "ROUND_CTX": round_len, "NKV_CTX": kk.shape[2],
                  "sliding_window_offset": 0, "sliding_window_size": int(n_local)}
        for name, t, axes in (("q", q, "zhmk"), ("k", kk, "zhnk"), ("v", vv, "zhkn"), ("o", o, "zhmn")):
            for axis, st in zip(axes, t.stride()):
                values[f"stride_{name}{axis}"] = st
        kern.launch_raw(values, ((N + 63) // 64, B * H))
        return kern

    keep = []
    if N > n_local:
        keep.append(stage("window", k, v))
        keep.append(stage("sink", k[:, :, :n_init].contiguous(), v[:, :, :n_init].contiguous()))
    else:
        keep.append(stage("single", k, v))
    torch.cuda.synchronize()          # the modules in `keep` must outlive their launches
    return o[:, :, :N].to(q.dtype)
