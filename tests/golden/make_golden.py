"""Writes tests/golden/qwen3_tiny_{a,b}.safetensors: logits of the reference engine's own CPU
path (aneesh-sathe/atomserve, unmodified) on tiny random models.

Run on a machine that has the reference checked out:

    python tests/golden/make_golden.py /path/to/atomserve

The reference needs Python 3.14 only for deferred annotations, so its files are compiled
here with the `annotations` future flag by an import hook; nothing in them is changed.
Weights come from tests/plain_qwen3.random_checkpoint (seeded) and are stored in the file
under `w.<tensor name>`, so that the test runs on exactly the weights the reference saw,
whatever random numbers the torch build at hand draws. Two ways of running are stored: every position of a whole prompt
(`whole`), and the same tokens as chunks of 7 next to single-token rows of a second
request (`mixed`), both through the reference's runner and paged pool.
"""

import __future__

import importlib.abc
import importlib.util
import pathlib
import sys

import torch
from safetensors.torch import save_file

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import plain_qwen3  # noqa: E402
from tiny_configs import TINY  # noqa: E402


def install_hook(ref: pathlib.Path) -> None:
    class Loader(importlib.abc.SourceLoader):
        def __init__(self, path):
            self.path = path

        def get_filename(self, name):
            return self.path

        def get_data(self, path):
            return pathlib.Path(path).read_bytes()

        def source_to_code(self, data, path, *, _optimize=-1):
            flag = __future__.annotations.compiler_flag
            return compile(data, path, "exec", flags=flag, dont_inherit=True)

    class Finder(importlib.abc.MetaPathFinder):
        def find_spec(self, name, path, target=None):
            if name != "atomserve" and not name.startswith("atomserve."):
                return None
            p = ref.joinpath(*name.split("."))
            if p.is_dir():
                init = str(p / "__init__.py")
                return importlib.util.spec_from_file_location(
                    name, init, loader=Loader(init), submodule_search_locations=[str(p)]
                )
            f = p.with_suffix(".py")
            if f.exists():
                return importlib.util.spec_from_file_location(name, f, loader=Loader(str(f)))
            return None

    sys.meta_path.insert(0, Finder())


def reference_weights(w: dict, cfg: dict):
    from atomserve.model import LayerWeights, Weights

    layers = []
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        layers.append(
            LayerWeights(
                input_norm=w[p + "input_layernorm.weight"],
                qkv_proj=torch.cat([w[p + f"self_attn.{n}_proj.weight"] for n in "qkv"]),
                q_norm=w[p + "self_attn.q_norm.weight"],
                k_norm=w[p + "self_attn.k_norm.weight"],
                o_proj=w[p + "self_attn.o_proj.weight"],
                post_attn_norm=w[p + "post_attention_layernorm.weight"],
                gate_up_proj=torch.cat([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]]),
                down_proj=w[p + "mlp.down_proj.weight"],
            )
        )
    embed = w["model.embed_tokens.weight"]
    head = embed if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return Weights(embed=embed, layers=layers, final_norm=w["model.norm.weight"], lm_head=head)


def prompts_for(cfg: dict, seed: int) -> tuple[list[int], list[int]]:
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(0, cfg["vocab_size"], (40,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab_size"], (9,), generator=g).tolist()
    return a, b


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <folder of the aneesh-sathe/atomserve checkout>")
    ref = pathlib.Path(sys.argv[1])
    install_hook(ref)
    from atomserve.config import ModelConfig
    from atomserve.kv_cache import KVPool
    from atomserve.runner import ModelRunner, Row

    for name in ("a", "b"):
        cfg, block_size = TINY[name]
        w = plain_qwen3.random_checkpoint(cfg, seed=11)
        mc = ModelConfig.from_dict(cfg)
        rw = reference_weights(w, cfg)
        ids, other = prompts_for(cfg, seed=5)
        # whole: one fresh prefill, logits at every position
        pool = KVPool(mc, 8, block_size, torch.device("cpu"), torch.float32)
        run = ModelRunner(rw, mc, pool)
        whole, _ = run.forward([Row(ids, 0, [6, 1, 4, 3, 7][: -(-40 // block_size)], num_logits=40)])
        # mixed: `ids` in chunks of 7 on scattered blocks, beside single tokens of `other`
        pool = KVPool(mc, 16, block_size, torch.device("cpu"), torch.float32)
        run = ModelRunner(rw, mc, pool)
        table_a = [9, 2, 11, 5, 14][: -(-40 // block_size)]
        table_b = [7, 0][: -(-9 // block_size)]
        got_a, got_b = [], []
        step = 0
        for start in range(0, 40, 7):
            chunk = ids[start : start + 7]
            rows = [Row(chunk, start, table_a, num_logits=len(chunk))]
            if step < len(other):
                rows.append(Row(other[step : step + 1], step, table_b, num_logits=1))
            logits, _ = run.forward(rows)
            got_a.append(logits[: len(chunk)])
            if step < len(other):
                got_b.append(logits[len(chunk) :])
            step += 1
        out = {
            "whole": whole.contiguous(),
            "mixed_a": torch.cat(got_a).contiguous(),
            "mixed_b": torch.cat(got_b).contiguous(),
            **{f"w.{k}": v.contiguous() for k, v in w.items()},
            "ids": torch.tensor(ids),
            "other": torch.tensor(other),
        }
        save_file(out, str(HERE / f"qwen3_tiny_{name}.safetensors"))
        print(name, {k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main()
