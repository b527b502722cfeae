"""The reference's benchmark configurations as model specs (shapes only; weights are seeded random draws)."""
from . import synth

CONFIGS = {
    # ReLU-Llama-2-7B shape, FP16, mean firing 10 %
    "relu-llama-7b-f16": dict(spec=synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.F16, n_layer=32, d=4096, n_ff=11008,
                                                   n_head=32, n_head_kv=32, rank=1024, n_vocab=32000, n_ctx=512, firing=0.10),
                              prompt=64, decode=128),
    # Falcon(ReLU)-40B shape, FP16
    "relu-falcon-40b-f16": dict(spec=synth.ModelSpec(arch=synth.ARCH_FALCON, wtype=synth.F16, n_layer=60, d=8192, n_ff=32768,
                                                     n_head=128, n_head_kv=8, rank=1024, n_vocab=65024, n_ctx=512, firing=0.10),
                                prompt=128, decode=256),
    # ReLU-Llama-2-70B shape, Q4_0 weights, FP16 predictors, mean firing 12 %: the configuration the headline metric is quoted on
    "relu-llama-70b-q4_0": dict(spec=synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.Q4_0, n_layer=80, d=8192, n_ff=28672,
                                                     n_head=64, n_head_kv=8, rank=1024, n_vocab=32000, n_ctx=768, firing=0.12),
                                prompt=256, decode=256),
    # OPT-175B shape, FP16 (needs >= 4 GPUs)
    "opt-175b-f16": dict(spec=synth.ModelSpec(arch=synth.ARCH_OPT, wtype=synth.F16, n_layer=96, d=12288, n_ff=49152,
                                              n_head=96, n_head_kv=96, rank=1536, n_vocab=50272, n_ctx=512, firing=0.08, norm_eps=0.0),
                         prompt=128, decode=128),
}
HEADLINE = "relu-llama-70b-q4_0"


def bytes_per_token(spec: synth.ModelSpec, active_per_layer: float) -> dict:
    """Algorithmic HBM bytes one decode step must read, per stage (whole model, all ranks): weights of ACTIVE rows only for
    the sparse FFN, dense weights elsewhere.  Row bytes: F16 2 cols, Q4_0 18 cols / 32."""
    rb = (lambda cols: cols // 32 * 18) if spec.wtype == synth.Q4_0 else (lambda cols: cols * 2)
    L, d, F, R = spec.n_layer, spec.d, spec.n_ff, spec.rank
    n_mats_updown = 2 if spec.arch == synth.ARCH_LLAMA else 1
    out = {
        "qkv": L * (d + 2 * spec.d_kv) * rb(d),
        "out_proj": L * d * rb(d),
        "predictor": L * 2 * R * (d + F),
        "up_gate": L * n_mats_updown * active_per_layer * rb(d),
        "down": L * active_per_layer * rb(d),
        "lm_head": spec.n_vocab * (rb(d) if spec.arch != synth.ARCH_OPT else 2 * d),
    }
    out["total"] = sum(out.values())
    out["sparse_ffn"] = out["up_gate"] + out["down"]        # the same bytes when one kernel does both (not added to the total twice)
    return out
