#!/usr/bin/env python3
"""Makes the golden logits: runs the reference project's own model code (its graph builder and
CPU executor, compiled here from its sources) on the two tiny random models of golden_model.py.

    python tests/golden/make_golden.py /path/to/reference [build_dir]

For each model it writes tests/golden/tiny_<name>.npz with the token ids, the logits of the whole
prompt (no cache) and the largest difference between that and a run in portions through the
reference's paged cache.  test_plain_model.py compares the plain implementation with these files,
so the plain implementation is anchored on the reference's code, not only on its formulas.
The reference needs its default -march=native build (include/minillm/runtime/kernels/cpu_simd.h:95).
"""
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from golden_model import GOLDEN_CONFIGS, golden_tokens, golden_weights  # noqa: E402

# checkpoint names -> the reference's graph constant names (src/model/transformer_graph_builder.cpp:140-205)
def reference_name(name: str) -> str:
    fixed = {"model.embed_tokens.weight": "tok_embeddings.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "lm_head.weight"}
    if name in fixed:
        return fixed[name]
    _, _, l, rest = name.split(".", 3)
    rest = (rest.replace("self_attn.", "").replace("mlp.", "").replace("input_layernorm", "attn_norm")
            .replace("post_attention_layernorm", "ffn_norm"))
    return f"layer_{l}.{rest}"


def main():
    ref = os.path.abspath(sys.argv[1])
    build = os.path.abspath(sys.argv[2]) if len(sys.argv) > 2 else tempfile.mkdtemp(prefix="ref_build_")
    if not os.path.exists(os.path.join(build, "libminillm_runtime.a")):
        subprocess.check_call(["cmake", "-S", ref, "-B", build, "-DCMAKE_BUILD_TYPE=Release", "-G", "Ninja"])
        subprocess.check_call(["ninja", "-C", build, "minillm_io"])
    driver = os.path.join(build, "reference_driver")
    libs = [os.path.join(build, f"libminillm_{n}.a") for n in ("io", "model", "runtime", "graph", "core")]
    subprocess.check_call(["g++", "-std=c++23", "-O2", "-march=native", "-I", os.path.join(ref, "include"),
                           os.path.join(HERE, "reference_driver.cpp"), *libs, "-o", driver])
    seed = 20240611
    for name, cfg in GOLDEN_CONFIGS.items():
        w = golden_weights(cfg, seed)
        toks = golden_tokens(cfg, seed)
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "in.bin")
            with open(path, "wb") as f:
                f.write(struct.pack("<10i", cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"],
                                    cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"],
                                    cfg["vocab_size"], int(cfg["tie_word_embeddings"]), len(toks), len(w)))
                f.write(struct.pack("<2d", cfg["rope_theta"], cfg["rms_norm_eps"]))
                f.write(toks.tobytes())
                for k, v in w.items():
                    b = reference_name(k).encode()
                    f.write(struct.pack("<i", len(b)) + b + struct.pack("<i", v.ndim) + struct.pack(f"<{v.ndim}i", *v.shape))
                    f.write(np.ascontiguousarray(v, dtype="<f4").tobytes())
            page = 16 if name == "A" else 8
            sizes = ["1"] if name == "A" else ["48", "2", "5", "1"]
            out = subprocess.check_output([driver, path, os.path.join(d, "whole.bin"), os.path.join(d, "por.bin"),
                                           str(page), "64", *sizes], text=True)
            V = cfg["vocab_size"]
            whole = np.fromfile(os.path.join(d, "whole.bin"), dtype="<f4").reshape(-1, V)
            por = np.fromfile(os.path.join(d, "por.bin"), dtype="<f4").reshape(-1, V)
        gap = float(np.abs(whole - por).max())
        np.savez_compressed(os.path.join(HERE, f"tiny_{name}.npz"), tokens=toks, logits=whole.astype(np.float32),
                            seed=np.int64(seed), whole_vs_portions=np.float32(gap))
        print(f"{name}: logits {whole.shape}, absmax {np.abs(whole).max():.3f}, whole vs portions {gap:.2e}; {out.strip()}")


if __name__ == "__main__":
    main()
