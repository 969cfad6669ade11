#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ with the reference's own model code.

    python tests/golden/make_golden.py --reference /path/to/cosmonomic-pulsar

It compiles ``golden_ref.cpp`` together with the reference's unchanged
``pulsar-core/src/model/qwen3.cpp``, ``paged_forward.cpp`` and
``runtime/kv/active_buffer.cpp`` for the CPU against the local libtorch, writes the tiny
random models A and B with this repository's random-weights mode, runs the reference's
``Qwen3Model::forward`` on one whole prompt each and stores the logits of a few positions
as ``tiny_<name>.json`` (token ids, positions, logits).  ``tests/test_plain.py`` regenerates
the same weights from the seed and compares the plain implementation with these files.

The reference's five CUDA ops are restated in ``golden_ref.cpp`` (the reference has no CPU
versions), so the golden files anchor the model code's structure (order of operations,
norm placement, residuals, head tying), not the arithmetic inside norm, rope or attention.
"""
import argparse
import json
import os
import struct
import subprocess
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import helpers  # noqa: E402

KEEP = 6          # positions kept per model (first, a few inside, last)


def compile_reference(reference: str, out: str) -> None:
    tdir = os.path.dirname(torch.__file__)
    core = os.path.join(reference, "pulsar-core")
    cmd = ["g++", "-std=c++23", "-O1", f"-I{core}/inc", f"-I{tdir}/include", f"-I{tdir}/include/torch/csrc/api/include",
           "-I/usr/local/cuda/include", os.path.join(HERE, "golden_ref.cpp"), f"{core}/src/model/qwen3.cpp",
           f"{core}/src/model/paged_forward.cpp", f"{core}/src/runtime/kv/active_buffer.cpp", f"-L{tdir}/lib", "-ltorch",
           "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", f"-Wl,-rpath,{tdir}/lib", "-o", out]
    print(" ".join(cmd))
    subprocess.run(cmd, check=True)


def dump_input(path: str, cfg: dict, weights: dict, tokens, page: int) -> None:
    untied = "lm_head.weight" in weights
    with open(path, "wb") as f:
        f.write(struct.pack("<10i", cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                            cfg["head_dim"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], int(untied),
                            page, len(tokens)))
        f.write(struct.pack("<2d", cfg["rope_theta"], cfg["rms_norm_eps"]))
        f.write(struct.pack(f"<{len(tokens)}i", *tokens))
        order = ["model.embed_tokens.weight", "model.norm.weight"]
        for i in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{i}."
            order += [p + n for n in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                                      "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                                      "self_attn.q_norm.weight", "self_attn.k_norm.weight", "mlp.gate_proj.weight",
                                      "mlp.up_proj.weight", "mlp.down_proj.weight")]
        if untied:
            order.append("lm_head.weight")
        for name in order:
            f.write(weights[name].float().contiguous().numpy().tobytes())


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "golden_ref")
        compile_reference(args.reference, exe)
        for name in ("A", "B"):
            raw, seed, page = helpers.TINY[name]
            folder = helpers.make_folder(os.path.join(tmp, name), raw, seed)
            cfg, weights = helpers.read_folder(folder)
            gen = torch.Generator().manual_seed(100 + seed)
            tokens = torch.randint(0, raw["vocab_size"], (24 if name == "A" else 40,), generator=gen).tolist()
            inp, outp = os.path.join(tmp, f"{name}.in"), os.path.join(tmp, f"{name}.out")
            dump_input(inp, cfg, weights, tokens, page)
            subprocess.run([exe, inp, outp], check=True)
            logits = torch.frombuffer(bytearray(open(outp, "rb").read()), dtype=torch.float32).view(len(tokens), -1)
            keep = sorted({0, 1, len(tokens) // 3, len(tokens) // 2, len(tokens) - 2, len(tokens) - 1})[:KEEP]
            with open(os.path.join(HERE, f"tiny_{name}.json"), "w") as f:
                json.dump({"config": name, "seed": seed, "tokens": tokens, "positions": keep,
                           "logits": [[round(float(x), 9) for x in logits[p]] for p in keep]}, f)
            print(f"tiny_{name}.json: positions {keep}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
