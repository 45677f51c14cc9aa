"""Checkpoint files in the reference's layout.

A checkpoint is a `torch.save` dict.  Keys (lm/train_340m/train_flagship.py:820-829,
lm/train_1p3b/train_hero_wave3d.py:738-745): `model` (plain `DualModLM.state_dict()`; the
RoPE tables are non-persistent buffers and therefore absent), `optimizer` (torch AdamW
layout), optional `optimizer_dm`, `step`, `applied`, `model_cfg` (= `DualModConfig.to_dict()`),
`gn_ema`, `gn_cnt`; the 1.3B trainer adds `engine_kwargs`, `wb_tick`, `clip_ema`, `tainted`,
`seed_offset`, `tokens`, `arch`.  Files: `ckpt_latest.pt` written atomically (temp + rename)
with the previous one kept as `ckpt_prev.pt`; `snap_%06d.pt`; `persist_%07d.pt` (model only).
`AsyncCheckpointWriter` snapshots tensors to host memory on the caller's thread and writes
the file on a worker thread (train_hero_wave3d.py:705-749).
"""

from __future__ import annotations

import os
import queue
import threading

import torch

from ..config import DualModConfig


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


def build_checkpoint(model, optimizer=None, *, step=0, applied=0, extra=None, optimizer_dm=None):
    ck = {"model": model.state_dict(), "step": int(step), "applied": int(applied),
          "model_cfg": model.cfg.to_dict()}
    if optimizer is not None:
        ck["optimizer"] = optimizer.state_dict()
    if optimizer_dm is not None:
        ck["optimizer_dm"] = optimizer_dm.state_dict()
    ck.update(extra or {})
    return ck


def save_atomic(ck, path, keep_prev=True):
    """Write `path` via a temp file + rename; the old file becomes `ckpt_prev.pt`."""
    d = os.path.dirname(os.path.abspath(path))
    os.makedirs(d, exist_ok=True)
    tmp = path + ".tmp"
    torch.save(ck, tmp)
    if keep_prev and os.path.exists(path):
        os.replace(path, os.path.join(d, "ckpt_prev.pt"))
    os.replace(tmp, path)


def save_checkpoint(out_dir, model, optimizer=None, *, step=0, applied=0, extra=None,
                    name="ckpt_latest.pt", optimizer_dm=None):
    ck = build_checkpoint(model, optimizer, step=step, applied=applied, extra=extra,
                          optimizer_dm=optimizer_dm)
    save_atomic(ck, os.path.join(out_dir, name), keep_prev=name == "ckpt_latest.pt")
    return ck


def save_snapshot(out_dir, ck, step):
    save_atomic(ck, os.path.join(out_dir, f"snap_{step:06d}.pt"), keep_prev=False)


def save_persist(out_dir, model, step, anchor=False, name=None):
    """Model-only file (`persist_%07d.pt` unless `name` is given); `anchor` also hard-links it as
    `anchor_%07d.pt`."""
    p = os.path.join(out_dir, name or f"persist_{step:07d}.pt")
    save_atomic({"model": model.state_dict(), "model_cfg": model.cfg.to_dict(), "step": int(step)},
                p, keep_prev=False)
    if anchor:
        a = os.path.join(out_dir, f"anchor_{step:07d}.pt")
        if not os.path.exists(a):
            os.link(p, a)
    return p


def load_checkpoint(path, map_location="cpu"):
    return torch.load(path, map_location=map_location, weights_only=False)


def model_from_checkpoint(ck, device="cpu", ctx_len=None, strict=True):
    """Rebuild the model a checkpoint describes.  `ctx_len` rebuilds the RoPE tables
    for a longer evaluation context (lm/eval/lm_eval_adapter.py:103-110)."""
    from ..models import DualModLM
    cfg = DualModConfig.from_dict(ck["model_cfg"])
    if ctx_len:
        cfg.max_seq_len = max(cfg.max_seq_len, ctx_len)
    model = DualModLM(cfg)
    model.load_state_dict(ck["model"], strict=strict)
    return model.to(device)


class AsyncCheckpointWriter:
    """Copies the checkpoint to host memory on the caller's thread (so training may go
    on mutating the live tensors) and serialises it on a worker thread.  At most one
    write is pending; `submit` waits for the previous one."""

    to_cpu = staticmethod(_to_cpu)      # host copy of a checkpoint dict (also used for resident snapshots)

    def __init__(self):
        self._q = queue.Queue(maxsize=1)
        self._err = None
        self._t = threading.Thread(target=self._loop, daemon=True)
        self._t.start()

    def _loop(self):
        while True:
            item = self._q.get()
            if item is None:
                return
            ck, path, keep_prev = item
            try:
                save_atomic(ck, path, keep_prev)
            except Exception as e:            # surfaced on the next submit / close
                self._err = e
            finally:
                self._q.task_done()

    def submit(self, ck, path, keep_prev=True):
        if self._err is not None:
            raise self._err
        self._q.join()
        self._q.put((_to_cpu(ck), path, keep_prev))

    def wait(self):
        self._q.join()
        if self._err is not None:
            raise self._err

    def close(self):
        self.wait()
        self._q.put(None)
