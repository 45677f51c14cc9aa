"""Configuration dataclasses.

`DualModConfig` carries every architecture / Dual-Mod knob of the reference
(models/dualmod/config.py:6-226) under the same field names, so a
`model_cfg` dict stored in a reference checkpoint rebuilds a model here with
`DualModConfig(**ck["model_cfg"])`.  `TrainConfig` mirrors the small-run
trainer settings (config.py:229-261).

Validation is table-driven: `_CHOICES` lists the legal values of every
enumerated knob, `_check_combinations` holds the cross-field rules.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, fields

_CHOICES = {
    "attn_mode": ("vanilla", "sequential", "deq", "static"),
    "gate_type": ("convex_sigmoid", "independent", "unbounded"),
    "gate_type_v": ("convex", "independent"),
    "gate_input": ("xu", "u", "x"),
    "gate_bias_init_k": ("scalar", "ugi", "committed"),
    "gate_bias_init_v": ("scalar", "ugi", "band"),
    "kmod_vraw_bound": ("none", "tanh"),
    "kmod_mode": ("raw", "gated_norm"),
    "v_norm": ("none", "rms"),
    "v_ctx_norm": ("none", "rms"),
    "k_ctx_norm": ("none", "rms"),
    "mlp_ratio": ("swiglu_8_3",),
    "ctx_mod": ("linear", "vmlp", "fusion", "kmlp", "puremlp", "puremlp_hw",
                "mult", "mult_res", "linpoint", "glu"),
    "dtype": ("bf16", "fp32", "fp16"),
}


@dataclass
class DualModConfig:
    # ---- trunk ----------------------------------------------------------
    d_model: int = 512
    n_layers: int = 8
    n_heads: int = 8
    n_kv_heads: int = 0             # 0 = MHA; fewer = GQA (vanilla path only)
    head_dim_override: int = 0      # 0 = d_model // n_heads (vanilla path only otherwise)
    vocab_size: int = 50257
    max_seq_len: int = 512
    local_window: int = 0           # W tokens including self; 0 = full causal
    rope_theta: float = 10000.0
    use_rope: bool = True           # False = NoPE (identity rotation)
    mlp_ratio: str = "swiglu_8_3"
    mlp_hidden_override: int = 0
    tie_embeddings: bool = True

    # ---- Dual-Mod write path -----------------------------------------------
    attn_mode: str = "sequential"
    enable_key_mod: bool = True
    enable_value_mod: bool = True
    gate_type: str = "convex_sigmoid"   # key gate (and legacy value gate) form
    gate_type_v: str = "convex"         # value gate: convex blend or two independent sigmoids
    gate_input: str = "xu"              # what the gates read: [x̂;u], u, or x̂
    gate_bias_init: float = 4.0
    gate_bias_init_k: str = "scalar"
    gate_bias_init_v: str = "scalar"
    ugi_eps: float = 0.04
    key_commit_bias: float = 3.0
    key_frontier_pairs: int = 6
    key_frontier_hi: float = 1.5
    value_band_lo: float = 0.2
    value_band_hi: float = 0.8
    ctx_reserved_init_std: float = 0.02
    gate_init_seed: int = 1337
    ctx_proj_init_std: float = 0.006
    rmsnorm_on_o: bool = True
    deq_sweeps: int = 4
    kmod_vraw_heads: int = 0            # first N heads: modulated keys, raw values
    ctx_mod: str = "linear"             # transition applied to u before w_vctx / w_kctx
    kmod_vraw_bound: str = "none"
    kmod_mode: str = "raw"
    gate_rank: int = 0                  # >0: gates factored in -> r -> out
    ctx_rank: int = 0                   # >0: ctx operators factored d -> r -> d
    v_norm: str = "none"                # per-head RMS of the raw value projection
    v_ctx_norm: str = "none"            # per-head RMS of the ctx value candidate
    mult_res_lambda: float = 1.0        # identity leak of the mult_res candidate
    k_ctx_norm: str = "none"            # per-head RMS (+gain) of the ctx key candidate
    attn_logn_ref: int = 0              # ln(n_keys)/ln(ref) logit scale; 0 = off
    k_gain_init: float = 1.75
    v_clamp_tau: float = 0.0            # per-(position, head) L2 cap on v''; 0 = off
    deterministic_bwd: bool = False     # engines: fixed-order gradient reductions

    # ---- training -------------------------------------------------------------
    checkpoint_chunk: int = 64          # scan re-materialisation granularity; 0 = off
    dtype: str = "bf16"

    def __post_init__(self):
        for name, legal in _CHOICES.items():
            val = getattr(self, name)
            if val not in legal:
                raise AssertionError(f"{name}={val!r} not in {legal}")
        self._check_combinations()

    def _check_combinations(self):
        if self.head_dim_override == 0:
            assert self.d_model % self.n_heads == 0, "d_model must divide into heads"
        kv = self.n_kv_heads_eff
        assert kv <= self.n_heads and self.n_heads % kv == 0, "bad n_kv_heads"
        if self.attn_mode != "vanilla":
            assert self.head_dim_override == 0 and self.n_kv_heads == 0, \
                "n_kv_heads / head_dim_override are vanilla-path only"
        structured = (self.gate_bias_init_k != "scalar"
                      or self.gate_bias_init_v != "scalar")
        if self.gate_rank > 0:
            assert not structured, \
                "structured gate-bias inits assume full-rank gate matrices"
        if self.ctx_rank > 0:
            assert self.gate_bias_init_k != "committed", \
                "committed key init writes dense W_Kctx rows; incompatible with ctx_rank"
            assert not self.ctx_mod.endswith("_hw"), \
                "_hw re-inits dense w_vctx; incompatible with ctx_rank"
        if self.kmod_mode == "gated_norm":
            assert self.kmod_vraw_bound == "none", \
                "kmod_vraw_bound applies to kmod_mode='raw' only"

    # ---- derived ----------------------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.head_dim_override or self.d_model // self.n_heads

    @property
    def n_kv_heads_eff(self) -> int:
        return self.n_kv_heads or self.n_heads

    @property
    def d_attn(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def mlp_hidden(self) -> int:
        if self.mlp_hidden_override:
            return self.mlp_hidden_override
        return int(round(self.d_model * 8 / 3 / 64) * 64)

    @property
    def gate_in_dim(self) -> int:
        return 2 * self.d_model if self.gate_input == "xu" else self.d_model

    @property
    def dual_mod_active(self) -> bool:
        return self.attn_mode != "vanilla" and (self.enable_key_mod or self.enable_value_mod)

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: dict) -> "DualModConfig":
        """Build from a stored dict, ignoring keys this version does not know."""
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})


@dataclass
class TrainConfig:
    run_name: str = "B-dualmod"
    out_dir: str = "out"
    data_dir: str = "data"
    batch_size: int = 128
    grad_accum: int = 1
    tokens_target: float = 300e6
    lr: float = 3e-4
    min_lr: float = 3e-5
    warmup_frac: float = 0.01
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    grad_clip: float = 1.0
    seed: int = 1337
    data_seed: int = 42
    log_interval: int = 10
    eval_interval: int = 250
    eval_iters: int = 32
    telemetry_interval: int = 500
    ckpt_interval: int = 2000
    wandb_log: bool = False
    wandb_project: str = "dualmod"
    compile: bool = False
    device: str = "cuda:0"

    def to_dict(self) -> dict:
        return asdict(self)


# ---- named shapes used by the benchmarks and trainers ---------------------------

def preset(name: str, **overrides) -> DualModConfig:
    """Named model shapes.

    `tiny_cpu`  1 layer d=128 (CPU exactness config)
    `a5_12m`    1 layer d=512 state-tracking model
    `dm_340m`   24 x d=1024, 16 heads x 64, ffn 2816, vocab 32000
    `dm_1p3b`   24 x d=2048, 16 heads x 128, ffn 5632, vocab 32000
    `hero_1p3b` the reference's 18 x d=2304 rank-144 mult_res recipe
                (engines/wave3d/config_1p3b.py:18-51)
    `dm_d960`   the reference's 340M run: 26 x d=960, 15 heads x 64, rank-120 mult_res write law, per-head key
                norm, one raw-pinned head, value clamp 150 (lm/train_340m/scripts/launch_dm_d960.sh:17-24)
    """
    shapes = {
        "tiny_cpu": dict(d_model=128, n_layers=1, n_heads=4, mlp_hidden_override=344,
                         vocab_size=64, max_seq_len=64, dtype="fp32", checkpoint_chunk=0),
        "a5_12m": dict(d_model=512, n_layers=1, n_heads=8, mlp_hidden_override=1376,
                       vocab_size=128, max_seq_len=256),
        "dm_340m": dict(d_model=1024, n_layers=24, n_heads=16, mlp_hidden_override=2816,
                        vocab_size=32000, max_seq_len=2048),
        "dm_1p3b": dict(d_model=2048, n_layers=24, n_heads=16, mlp_hidden_override=5632,
                        vocab_size=32000, max_seq_len=4096),
        "hero_1p3b": dict(d_model=2304, n_layers=18, n_heads=36, vocab_size=32000,
                          max_seq_len=4096, ctx_mod="mult_res", gate_rank=144, ctx_rank=144,
                          k_ctx_norm="rms", kmod_vraw_heads=1, v_clamp_tau=150.0,
                          gate_bias_init=4.0),
        "dm_d960": dict(d_model=960, n_layers=26, n_heads=15, vocab_size=32000, max_seq_len=2048,
                        ctx_mod="mult_res", gate_rank=120, ctx_rank=120, k_ctx_norm="rms", k_gain_init=1.75,
                        kmod_vraw_heads=1, v_clamp_tau=150.0, gate_bias_init=0.0),
    }
    kw = dict(shapes[name])
    kw.update(overrides)
    return DualModConfig(**kw)
