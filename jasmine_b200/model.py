"""Host-side handle of the decoder-only model of libjasmine_b200.so (jsm_llama_*), for tests and bench.py."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import ALLREDUCE_FN, BF16, F32, ModelConfig, check, lib, stream_ptr


class Llama:
    def __init__(self, n_layers, d_model, n_heads, n_kv_heads, d_ffn, vocab, max_batch, max_context, head_dim=128,
                 norm_eps=1e-5, rope_theta=10000.0, seed=4, tp_rank=0, tp_size=1, pool_pages=0):
        """pool_pages > 0: continuous batching (jsm_llama_create_paged): admit / step_active / retire."""
        self.cfg = ModelConfig(n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ffn, vocab, max_batch, max_context,
                               norm_eps, rope_theta, tp_rank, tp_size)
        self._h = C.c_void_p()
        if pool_pages > 0:
            check(lib().jsm_llama_create_paged(C.byref(self.cfg), seed, pool_pages, C.byref(self._h)))
        else:
            check(lib().jsm_llama_create(C.byref(self.cfg), seed, C.byref(self._h)))
        self._cb = None

    # ---- continuous batching (host tensors in, host values out) ----
    def admit(self, h_prompt, h_logits_last=None):
        """Prefills a prompt (int32 host tensor) into the next free batch row; returns (row, first generated token)."""
        row, tok = C.c_int(), C.c_int32()
        check(lib().jsm_llama_seq_admit(self._h, h_prompt.data_ptr(), h_prompt.numel(), C.byref(row), C.byref(tok),
                                        h_logits_last.data_ptr() if h_logits_last is not None else None, stream_ptr()))
        return row.value, tok.value

    def step_active(self, h_ids, h_next, h_logits=None):
        check(lib().jsm_llama_step_active(self._h, h_ids.data_ptr(), h_next.data_ptr(),
                                          h_logits.data_ptr() if h_logits is not None else None, stream_ptr()))

    def retire(self, row: int) -> int:
        """Frees the row; returns the old index of the row that moved into its place, or -1."""
        moved = C.c_int()
        check(lib().jsm_llama_seq_retire(self._h, row, C.byref(moved), stream_ptr()))
        return moved.value

    def pool_state(self):
        a, f, t = C.c_int(), C.c_int(), C.c_int()
        check(lib().jsm_llama_pool_state(self._h, C.byref(a), C.byref(f), C.byref(t)))
        return a.value, f.value, t.value

    def close(self):
        if self._h:
            check(lib().jsm_llama_destroy(self._h))
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_allreduce(self, fn):
        """fn(ptr, count, dtype, stream) sums in place across the tensor-parallel group."""
        def tramp(ptr, count, dtype, stream, _user):
            try:
                fn(ptr, count, dtype, stream)
                return 0
            except Exception:  # the library reports JSM_NCCL
                import traceback
                traceback.print_exc()
                return 1
        self._cb = ALLREDUCE_FN(tramp)
        check(lib().jsm_llama_set_allreduce(self._h, self._cb, None))

    def connect_peers(self, dist) -> None:
        """Makes the exchange regions of all ranks of one node addressable from this rank (CUDA IPC handles passed
        through torch.distributed) and switches the model to its own all-reduce over peer memory."""
        rank, world = self.cfg.tp_rank, self.cfg.tp_size
        p, n = C.c_void_p(), C.c_size_t()
        check(lib().jsm_llama_tp_region(self._h, C.byref(p), C.byref(n)))
        handle = C.create_string_buffer(64)
        check(lib().jsm_ipc_export(p, handle))
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw)
        ptrs = (C.c_void_p * world)()
        self._peer_ptrs = []
        for r in range(world):
            if r == rank:
                ptrs[r] = p.value
                continue
            q = C.c_void_p()
            check(lib().jsm_ipc_import(C.create_string_buffer(handles[r], 64), C.byref(q)))
            ptrs[r] = q.value
            self._peer_ptrs.append(q)
        check(lib().jsm_llama_tp_connect(self._h, ptrs))
        dist.barrier()

    def weight(self, name: str) -> np.ndarray:
        """A weight of this rank's shard as float32 (bf16 tensors are widened)."""
        p, n = C.c_void_p(), C.c_size_t()
        check(lib().jsm_llama_weight(self._h, name.encode(), C.byref(p), C.byref(n)))
        is_f32 = name.endswith(("g1", "g2", "gf"))
        buf = np.empty(n.value, np.float32 if is_f32 else np.uint16)
        check(lib().jsm_download(buf.ctypes.data, p, buf.nbytes, stream_ptr()))
        if is_f32:
            return buf
        return (buf.astype(np.uint32) << 16).view(np.float32)

    def set_weight(self, name: str, tensor):
        """Replaces a tensor of this rank's shard from a CUDA tensor (bf16 row-major [out, in]; gains f32 [d])."""
        check(lib().jsm_llama_set_weight(self._h, name.encode(), tensor.data_ptr(), tensor.numel(), stream_ptr()))

    def save(self, path: str):
        check(lib().jsm_llama_save(self._h, str(path).encode()))

    def load(self, path: str):
        check(lib().jsm_llama_load(self._h, str(path).encode()))

    def prefill(self, ids, seq: int, next_tokens=None, logits_last=None):
        check(lib().jsm_llama_prefill(self._h, ids.data_ptr(), seq, ids.numel(),
                                      next_tokens.data_ptr() if next_tokens is not None else None,
                                      logits_last.data_ptr() if logits_last is not None else None, stream_ptr()))

    def decode_step(self, ids, next_tokens, logits=None):
        check(lib().jsm_llama_decode_step(self._h, ids.data_ptr(), ids.numel(), next_tokens.data_ptr(),
                                          logits.data_ptr() if logits is not None else None, stream_ptr()))

    def decode_step_host(self, h_ids, h_next, h_logits=None):
        """jsm_llama_decode_step_host: token ids from a host tensor (pinned for speed), next tokens into a host tensor;
        returns after the outputs are valid."""
        check(lib().jsm_llama_decode_step_host(self._h, h_ids.data_ptr(), h_ids.numel(), h_next.data_ptr(),
                                               h_logits.data_ptr() if h_logits is not None else None, stream_ptr()))

    def set_context(self, seq: int, n: int):
        check(lib().jsm_llama_set_context(self._h, seq, n))

    def reset(self):
        check(lib().jsm_llama_reset(self._h))

    def step_bytes(self):
        w, k = C.c_uint64(), C.c_uint64()
        check(lib().jsm_llama_step_bytes(self._h, C.byref(w), C.byref(k)))
        return w.value, k.value
