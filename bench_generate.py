"""Whole-generation benchmark in the shape of the reference's summarize.py (summarize.py:29-145).

    python bench_generate.py [--model opt-1.3b|gpt-j-6b] [--prompt 1000] [--output-len 256] [--samples 20]

The reference times `model.generate` of a HuggingFace OPT / GPT-J over cnn_dailymail articles for
batch sizes 1, 2, 5, 10 with three attention implementations (summarize.py:82-96: HuggingFace's own,
FFA with its measured launch, FFA with the FasterTransformer launch) and prints the summed
wall-clock seconds per (implementation, batch size) (summarize.py:126-141; README.md:51-65).
Model weights, the dataset and the rouge metric are not available offline, so this script keeps the
LOOP and replaces the inputs: a decoder of the same architecture (layers, width, heads, FFN,
vocabulary) with seeded random fp16 weights, random token ids of the stated prompt length, greedy
decoding for a fixed number of new tokens.  Per-generate wall-clock with a device sync on both
sides, summed over samples/batch generations, as the reference does.  Three implementations:

  torch          keys and values grow by torch.cat, attention = softmax(q K^T) V with bmm -- what the
                 HuggingFace model does without FFA (modeling_opt.py:228-262)
  engine         one FastForwardAttn per layer built from the prompt's K/V, one attention call per
                 layer per token -- how the reference's fork drives FFA (modeling_opt.py:201-226)
  engine-graph   the same engines, all layers of a token recorded once in a CUDA graph (GraphedLayers)

Absolute seconds are not comparable with README.md:51-65 (random weights, no tokenizer, another GPU);
the ratios between the rows are the result.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {   # layers, width, heads, FFN width, vocabulary, positions (facebook/opt-1.3b, EleutherAI/gpt-j-6b configs)
    "opt-1.3b": dict(layers=24, width=2048, heads=32, ffn=8192, vocab=50272, positions=2050),
    "gpt-j-6b": dict(layers=28, width=4096, heads=16, ffn=16384, vocab=50400, positions=2048),
}


class Decoder:
    """Pre-LayerNorm decoder with learned positions (the OPT block; GPT-J's parallel block and
    rotary positions change nothing in the attention call, so the same block stands in for it)."""

    def __init__(self, cfg, dtype, dev, seed=0):
        g = torch.Generator(device=dev).manual_seed(seed)
        E, Fw = cfg["width"], cfg["ffn"]
        self.cfg, self.dtype, self.dev = cfg, dtype, dev
        self.H, self.Dh = cfg["heads"], E // cfg["heads"]

        def w(*shape, std):
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).to(dtype)

        self.tok = w(cfg["vocab"], E, std=0.02)
        self.pos = w(cfg["positions"], E, std=0.02)
        self.layers = [dict(qkv=w(E, 3 * E, std=E ** -0.5), out=w(E, E, std=E ** -0.5 / (2 * cfg["layers"]) ** 0.5),
                            fc1=w(E, Fw, std=E ** -0.5), fc2=w(Fw, E, std=Fw ** -0.5 / (2 * cfg["layers"]) ** 0.5))
                       for _ in range(cfg["layers"])]

    def mlp(self, L, x):
        return x + F.relu(F.layer_norm(x, x.shape[-1:]) @ L["fc1"]) @ L["fc2"]

    def qkv(self, L, x):
        """x [B, T, E] -> q (pre-scaled, modeling_opt.py:182), k, v as [B, H, T, Dh]."""
        B, T, E = x.shape
        q, k, v = (F.layer_norm(x, (E,)) @ L["qkv"]).split(E, dim=-1)
        shape = lambda a: a.view(B, T, self.H, self.Dh).transpose(1, 2)
        return shape(q) * self.Dh ** -0.5, shape(k), shape(v)

    def prefill(self, ids):
        """Prompt pass.  Returns the last position's hidden state [B, E] and every layer's K, V [B, H, T, Dh]."""
        B, T = ids.shape
        x = self.tok[ids] + self.pos[2:T + 2]
        kvs = []
        for L in self.layers:
            q, k, v = self.qkv(L, x)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0)
            x = x + a.transpose(1, 2).reshape(B, T, -1) @ L["out"]
            x = self.mlp(L, x)
            kvs.append((k.contiguous(), v.contiguous()))
        return x[:, -1], kvs

    def next_token(self, h):
        return (F.layer_norm(h, h.shape[-1:]) @ self.tok.t()).argmax(-1)


def generate(model, ids, new_tokens, impl):
    from fastforwardattention_b200 import FastForwardAttn, GraphedLayers

    B, T = ids.shape
    E, H, Dh = model.cfg["width"], model.H, model.Dh
    h, kvs = model.prefill(ids)
    out = [model.next_token(h)]
    if impl == "torch":
        Ks, Vs = [k for k, _ in kvs], [v for _, v in kvs]
        for s in range(new_tokens - 1):
            x = (model.tok[out[-1]] + model.pos[T + s + 2])[:, None]
            for i, L in enumerate(model.layers):
                q, k, v = model.qkv(L, x)
                Ks[i], Vs[i] = torch.cat([Ks[i], k], 2), torch.cat([Vs[i], v], 2)     # modeling_opt.py:228-230
                w = torch.softmax(torch.matmul(q, Ks[i].transpose(-1, -2)), dim=-1)
                x = x + torch.matmul(w, Vs[i]).transpose(1, 2).reshape(B, 1, E) @ L["out"]
                x = model.mlp(L, x)
            out.append(model.next_token(x[:, 0]))
        return torch.stack(out, 1)
    engines = [FastForwardAttn(k, v, T + new_tokens, False) for k, v in kvs]            # modeling_opt.py:219-220
    del kvs
    if impl == "engine":
        for s in range(new_tokens - 1):
            x = (model.tok[out[-1]] + model.pos[T + s + 2])[:, None]
            for i, L in enumerate(model.layers):
                q, k, v = model.qkv(L, x)
                a = engines[i].attention(q, k, v, 1.0, T + s, 0.0)                     # modeling_opt.py:203
                x = x + a.reshape(B, 1, E) @ L["out"]
                x = model.mlp(L, x)
            out.append(model.next_token(x[:, 0]))
        return torch.stack(out, 1)
    # engine-graph: embedding, all layers, the next-token choice and the position counter in one graph
    position = torch.full((1,), T + 2, dtype=torch.int64, device=ids.device)

    def body(tok, attend):
        x = (model.tok[tok] + model.pos[position])[:, None]
        for i, L in enumerate(model.layers):
            q, k, v = model.qkv(L, x)
            x = x + attend(i, q, k, v).reshape(B, 1, E) @ L["out"]
            x = model.mlp(L, x)
        position.add_(1)
        return model.next_token(x[:, 0])

    step = GraphedLayers(engines, 1.0, first_row=T, body=body, example_input=out[-1])
    position.fill_(T + 2)   # the warm-up trace inside the constructor advanced it once
    for s in range(new_tokens - 1):
        out.append(step(out[-1]).clone())
    return torch.stack(out, 1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="opt-1.3b", choices=sorted(MODELS))
    ap.add_argument("--prompt", type=int, default=1000)      # summarize.py:60 keeps the last 1000 words
    ap.add_argument("--output-len", type=int, default=256)   # README.md:48
    ap.add_argument("--samples", type=int, default=20, help="articles per batch size (the reference's --max_ite)")
    ap.add_argument("--batch-sizes", default="1,2,5,10")     # summarize.py:82
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    model = Decoder(MODELS[args.model], torch.float16, dev)
    impls = ["torch", "engine", "engine-graph"]
    rows, agree = {i: {} for i in impls}, {}
    with torch.no_grad():
        for bs in [int(x) for x in args.batch_sizes.split(",")]:
            n_gen = max(1, args.samples // bs)
            g = torch.Generator(device=dev).manual_seed(bs)
            batches = [torch.randint(4, model.cfg["vocab"], (bs, args.prompt), generator=g, device=dev) for _ in range(n_gen)]
            tokens = {}
            for impl in impls:
                generate(model, batches[0], 8, impl)   # warm-up: library handles, kernel attributes
                total = 0.0
                for ids in batches:
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                    toks = generate(model, ids, args.output_len, impl)
                    torch.cuda.synchronize()
                    total += time.perf_counter() - t0
                tokens[impl] = toks
                rows[impl][bs] = round(total, 3)
            # greedy choices of the last generation: identical prefix length (random weights give near-ties,
            # after the first differing token the continuations are different sequences)
            same = [int(((tokens["torch"] == tokens[i]).int().cumprod(1).sum(1).float().mean()).item()) for i in impls[1:]]
            agree[bs] = {"engine": same[0], "engine-graph": same[1], "of": args.output_len}
    line = {"benchmark": "generate", "model_shape": args.model, "dtype": "f16", "weights": "seeded random", "prompt_tokens": args.prompt,
            "new_tokens": args.output_len, "samples_per_batch_size": args.samples, "unit": "seconds summed over samples/batch generations",
            "seconds": rows, "speedup_vs_torch": {i: {bs: round(rows["torch"][bs] / rows[i][bs], 2) for bs in rows[i]} for i in impls[1:]},
            "tokens_identical_to_torch_up_to": agree}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
