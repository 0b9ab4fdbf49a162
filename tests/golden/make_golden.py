"""Generate the golden fixtures in this directory from the reference itself.

Run where a checkout of the reference exists; give its path as the argument or in the
REFERENCE_ROOT environment variable:

    python tests/golden/make_golden.py <path to the better-benchmark checkout>

For every case below the script loads the reference's own ``Repro`` module from
``repros/canonical/<dir>/repro.py``, builds inputs with the reference's own
``repro_harness.make_inputs_from_config`` (seed 1, CPU, at a reduced shape written in the
reference's compact shapes.json encoding), runs the module, and also records the reference's
``byte_accounting.count_bytes_effective`` for the same call. Inputs, outputs and byte count go to
``<case>.pt``. Nothing from the reference is copied: only tensors it computed are stored.
"""
import os
import sys
from pathlib import Path

import torch

_root = os.environ.get("REFERENCE_ROOT") or (sys.argv[1] if len(sys.argv) > 1 else "")
if not _root:
    raise SystemExit("usage: make_golden.py <path to the reference checkout>  (or set REFERENCE_ROOT)")
REFERENCE_ROOT = Path(_root)
HERE = Path(__file__).resolve().parent

# case name -> (canonical dir in the reference, compact input entries at a reduced shape)
CASES = {
    "ln_fwd_f8ec553e339e": ("var_mean_f8ec553e339e",
                            [[[4, 24, 320], "f32"], [[320], "f32"], [[320], "f32"], ["S", [96, 320]]]),
    "rmsnorm_fwd_f667cd8901af": ("mean_f667cd8901af", [[[96, 512], "bf16"], [[512], "f32"]]),
    "softmax_bias_20ccc18dda60": ("amax_sum_20ccc18dda60",
                                  [[[32, 16, 64], "bf16"], [[4, 1, 16, 64], "bf16"],
                                   ["S", [4, 8, 16, 64]], ["S", [32, 16, 64]]]),
    "bn_relu_42fad1ece813": ("var_mean_42fad1ece813",
                             # N*H*W stays 8192: the captured graph hard-codes the unbiasing factor 8192/8191
                             [[[128, 8, 8, 8], "bf16", {"st": [512, 1, 64, 8]}], [[8], "f32"],
                              [[8], "f32"], [[8], "f32"], [[8], "f32"]]),
    "rms_bwd_2cd99e5eb23e": ("sum_sum_2cd99e5eb23e",
                             # the row length stays 512: the captured graph hard-codes it as a divisor
                             [[[], "bf16"], [[512], "f32"], [[60, 1], "f32"], [[60, 512], "bf16"],
                              ["S", [60, 512]], ["S", [60, 512]], ["S", [512]]]),
    "ln_bwd_3cac3bbf4e8f": ("sum_sum_sum_3cac3bbf4e8f",
                            [[[60, 1], "f32"], [[], "bf16"], [[512], "f32"], [[60, 512], "bf16"],
                             [[60, 1], "f32"], ["S", [60, 512]]]),
    "colsum_eb86a17deab9": ("sum_eb86a17deab9", [[[4, 48, 160], "f32"]]),
    "headsplit_c0d19d490a2f": ("pointwise_c0d19d490a2f",
                               [[[64, 96], "bf16"], ["S", [4, 16, 96]], ["S", [4, 16, 3, 32]],
                                ["S", [12, 16, 32]]]),
    "transpose_021e90d9c17d": ("pointwise_021e90d9c17d", [[[4, 3, 49, 32], "bf16"], ["S", [4, 96, 7, 7]]]),
    "logsoftmax_d16035e7b826": ("amax_sum_d16035e7b826", [[[24, 520], "bf16"], ["S", [2, 12, 517]]]),
    "softmax_long_7079889cfc04": ("amax_sum_7079889cfc04", [[[6, 5000], "bf16"]]),
    "bn_bwd_leaky_12fc8ebf8180": ("sum_sum_12fc8ebf8180",
                                  # N*H*W stays 8192: the captured graph hard-codes 1/8192
                                  [[[32, 8, 16, 16], "bf16"], [[32, 8, 16, 16], "bf16"], [[32, 8, 16, 16], "bf16"],
                                   [[1, 8, 1, 1], "f32"], [[8], "f32"], [[8], "f32"]]),
    "spatial_mean_c9e1a8113328": ("mean_c9e1a8113328", [[[4, 48, 5, 5], "bf16", {"st": [1200, 1, 240, 48]}]]),
    # two dropout masks drawn inside the region: the masks are outputs, so the recorded run fixes them
    "dropout_rms_014afd4984e6": ("mean_014afd4984e6",
                                 [[[64, 512], "bf16"], [[84], "i64"], [[2, 32, 512], "f32"], [[512], "f32"],
                                  ["S", [2, 32, 512]], ["S", [2, 32, 512]], ["S", [2, 32, 512]], ["S", [64, 512]]]),
    # the row length stays 768: the captured graph hard-codes it as a divisor
    "dropout_ln_01fbd6c1b27f": ("var_mean_01fbd6c1b27f",
                                [[[64, 768], "bf16"], [[36], "i64"], [[2, 32, 768], "f32"], [[768], "f32"],
                                 [[768], "f32"], ["S", [2, 32, 768]], ["S", [2, 32, 768]]]),
    "gelu_ln_af505388b035": ("var_mean_af505388b035",
                             [[[96, 768], "bf16"], [[768], "bf16"], [[768], "bf16"], ["S", [4, 24, 768]], ["S", [96, 768]]]),
    # outputs that are views: values here, the aliasing structure in tests/test_gpu_aliasing.py
    "cast_alias_8bb40810003c": ("pointwise_8bb40810003c", [[[40, 96], "f32"]]),
    "scale_view_95ed2ef35da9": ("pointwise_95ed2ef35da9",
                                [[[64, 96], "bf16"], ["S", [4, 16, 96]], ["S", [4, -1, 3, 32]]]),
    # the packed width stays 3 * 768: the captured graph splits at the literal 768
    "qkv_views_1611fb0c7845": ("pointwise_1611fb0c7845",
                               [[[32, 2304], "bf16"], ["S", [2, 16, 2304]], ["S", [2, 16, 12, 64]],
                                ["S", [2, 16, 12, 64]], ["S", [2, 16, 12, 64]]]),
    "headmerge_e87d6ebc9ded": ("pointwise_e87d6ebc9ded",
                               [[[12, 16, 32], "bf16"], ["S", [4, 3, 16, 32]], ["S", [4, -1, 96]], ["S", [64, 96]]]),
    # returned as k, v, q; the packed width stays 3 * 768 (the graph splits at the literal 768)
    "qkv_views_d5a413a2c233": ("pointwise_d5a413a2c233",
                               [[[32, 2304], "bf16"], ["S", [2, 16, 2304]], ["S", [2, 16, 12, 64]],
                                ["S", [2, 16, 12, 64]], ["S", [2, 16, 12, 64]]]),
    "gelu_ln_stats_21faaccf749d": ("var_mean_21faaccf749d",
                                   [[[96, 768], "bf16"], [[768], "f32"], [[768], "f32"], ["S", [4, 24, 768]], ["S", [96, 768]]]),
    # the bias is handed over permuted (head dimension unit-stride), as in the captured shape point
    "softmax_dropout_089fdab8f22b": ("amax_sum_089fdab8f22b",
                                     [[[12, 16, 64], "bf16"], [[4, 3, 16, 64], "f32", {"st": [3072, 1, 192, 3]}],
                                      [[84], "i64"], ["S", [4, 3, 16, 64]], ["S", [4, 3, 16, 64]],
                                      ["S", [4, 3, 16, 64]], ["S", [12, 16, 64]]]),
    # residual add -> LayerNorm and four of its siblings (other eps, other outputs, fp32 weights)
    "res_ln_0ada225c0a04": ("var_mean_0ada225c0a04",
                            [[[96, 768], "bf16"], [[4, 24, 768], "bf16"], [[768], "bf16"], [[768], "bf16"],
                             ["S", [4, 24, 768]], ["S", [96, 768]]]),
    "res_ln_sum_f4578c128d74": ("var_mean_f4578c128d74",
                                [[[66, 320], "bf16"], [[2, 33, 320], "bf16"], [[320], "bf16"], [[320], "bf16"],
                                 ["S", [2, 33, 320]], ["S", [66, 320]]]),
    "res_ln_alias_45f7dfd4a983": ("var_mean_45f7dfd4a983",
                                  [[[24, 4096], "bf16"], [[2, 12, 4096], "bf16"], [[4096], "bf16"], [[4096], "bf16"],
                                   ["S", [2, 12, 4096]], ["S", [24, 4096]]]),
    "res_ln_sum2_49afc8635b79": ("var_mean_49afc8635b79",
                                 [[[96, 768], "bf16"], [[4, 24, 768], "bf16"], [[768], "bf16"], [[768], "bf16"],
                                  ["S", [4, 24, 768]], ["S", [-1, 768]]]),
    "res_ln_stats_547bcc63004b": ("var_mean_547bcc63004b",
                                  [[[80, 240], "bf16"], [[5, 16, 240], "bf16"], [[240], "f32"], [[240], "f32"],
                                   ["S", [5, 16, 240]], ["S", [80, 240]]]),
    # parameter casts (a channels-last weight keeps its strides) and ReLU, all in storage order
    "cast_param_04d85912d998": ("pointwise_04d85912d998", [[[8, 3, 3, 3], "bf16", {"st": [27, 1, 9, 3]}]]),
    "cast_param_ccd411f2a45d": ("pointwise_ccd411f2a45d", [[[1003], "f32"]]),
    "relu_3abc926270f6": ("pointwise_3abc926270f6", [[[4, 24, 5, 5], "bf16"]]),
    "gelu_826ea0b5f6e4": ("pointwise_826ea0b5f6e4", [[[66, 96], "bf16"], ["S", [2, 33, 96]], ["S", [66, 96]]]),
    "silu_795cdbe23b17": ("pointwise_795cdbe23b17", [[[4, 24, 9, 9], "bf16", {"st": [1944, 1, 216, 24]}]]),
    "dropout_add_4b076ed1ff41": ("pointwise_4b076ed1ff41",
                                 [[[48, 320], "bf16"], [[2], "i64"], [[3, 16, 320], "f32"],
                                  ["S", [3, 16, 320]], ["S", [3, 16, 320]]]),
}


def main():
    sys.path.insert(0, str(REFERENCE_ROOT))
    sys.path.insert(0, str(REFERENCE_ROOT / "scripts"))
    import byte_accounting
    import input_codec
    import oracle_harness
    import repro_harness

    def build_inputs(compact):
        specs = [input_codec.spec_from_compact(e) for e in compact]
        for s in specs:
            if s.get("kind") == "tensor":
                s["device"] = "cpu"
        torch.manual_seed(1)
        return repro_harness.make_inputs_from_config({"inputs": specs})

    for name, (dirname, compact) in CASES.items():
        repro_dir = REFERENCE_ROOT / "repros" / "canonical" / dirname
        module = oracle_harness.load_repro_module(repro_dir)
        inputs = build_inputs(compact)
        with torch.no_grad():
            outputs = module.Repro()(*build_inputs(compact))
        nbytes = byte_accounting.count_bytes_effective(module.Repro(), build_inputs(compact))
        flat = oracle_harness._normalize_outputs(outputs)
        torch.save({"reference_dir": dirname, "compact_inputs": compact, "inputs": inputs,
                    "outputs": [o.clone() for o in flat], "effective_bytes": int(nbytes),
                    "torch_version": torch.__version__}, HERE / f"{name}.pt")
        print(f"{name}: {len(flat)} outputs, {nbytes} bytes")


if __name__ == "__main__":
    main()
