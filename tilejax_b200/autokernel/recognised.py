"""Fingerprints (fingerprint.py) of the loop nests the attention and decode kernels accept, by family.

Written by `python -m tilejax_b200.autokernel.fingerprint [reference/examples]`: the forms in this package's
kernels.py and, when the reference's example files are at hand, the forms in examples/causal_attention.py,
examples/decode.py, examples/rmsnorm_matmul.py, examples/attention_block.py and
examples/ragged_paged_attention.py (lane-replicated row statistics, block-diagonal queries, paired words).
Do not edit by hand."""

RECOGNISED: dict[str, dict[str, str]] = {
    "attention": {
        "c0907b9932813d96d8d5d1f74db165d93c89872bf5fd1650ac21326ccad72e03": "examples/causal_attention.py causal_attention",
        "dffc41f8367fc51d53b1060ab8009f21a063452afd282a1bc6d325036bca8e97": "tilejax_b200/autokernel/kernels.py causal_attention",
    },
    "attention_block": {
        "7ef581c0a492777f44e2645bb412d36121f2fb4a0b2ade0d8fa6f96a66531503": "examples/attention_block.py attention_block",
        "a0d794a17081d7572269488d57098f6abb0aa4e8683247f5daa1f64fe00e94d6": "tilejax_b200/autokernel/kernels.py attention_block",
    },
    "decode": {
        "51a65e439275a796e84d550d1efbeca191aa4c8dcadf30cddde5bacac4a58c87": "examples/decode.py gqa_decode",
        "ce6c35ee904aa743e268168c44b35ae4d64e545a5b1fb7d672b9187c1434147e": "examples/decode.py paged_gqa_decode",
        "9f93df037dfb1451472f851a52f91a9008e3db6637d8b62a8964fffc10d6bfef": "tilejax_b200/autokernel/kernels.py gqa_decode",
        "897c9c9ab27439d4820244e1191ff336b32075fe8275a78a9ab02fcba97f16ad": "tilejax_b200/autokernel/kernels.py paged_gqa_decode",
    },
    "mla": {
        "8040e261b18bb83fef376fc89112926911a5d9cb73e4c2b39e44d2ae6d5aaa26": "examples/decode.py mla_decode",
        "63bc9dae7ce3b319b7958f67d95b958eb7131acaa7f7f993789d798a913dcbd5": "tilejax_b200/autokernel/kernels.py mla_decode",
    },
    "rmsnorm": {
        "ebbdf02fc35cd281f7cba2fdd95589e0d8717f3476647b2313b8393a40b81e26": "examples/rmsnorm_matmul.py rmsnorm_matmul",
        "bc7e5bbddff3f245c47e9cbeea906d10d142f2fe1e7f9fd7b4a7eeb32f1c031d": "tilejax_b200/autokernel/kernels.py rmsnorm_matmul",
    },
    "rpa_decode": {
        "9c7c8eadbba15db816b68fdb97c1db23c79f3bd0271a905b33d9cc1f13b2ace2": "examples/ragged_paged_attention.py make_decode",
        "696fd4feefd3a8683940cba797e0bab498b59e7d6d01532804293f16acfa9fe4": "tilejax_b200/autokernel/kernels.py make_rpa_decode",
    },
    "rpa_prefill": {
        "cbaa8046c2a0deb3deedebe1db8dad7806c5cd06e62a0ed9662d5a627fc5f8d0": "examples/ragged_paged_attention.py make_prefill",
        "0fce51cce7ad19b9991a5e8051ac449fa8804e234a5e9cee9a155610c3621781": "tilejax_b200/autokernel/kernels.py make_rpa_prefill",
    },
    "rpa_write": {
        "def963b42a5c366a39776b84afb2a63038a660fb73310acbfba03d1e39d81308": "examples/ragged_paged_attention.py rpa_write",
        "3fee2d20ba0172da09fb01183ac7ab746c160528b82cd1c3bd876fd6046eba06": "tilejax_b200/autokernel/kernels.py rpa_write",
    },
}
