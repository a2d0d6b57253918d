#!/usr/bin/env python3
"""Command line: generate from a model folder on one GPU.

Option names follow the reference's scripts where it has them: ``--model``, ``--prompt``,
``--sampler-temp``, ``--sampler-top-p``, ``--sampler-top-k`` (main.py:9-25); ``--max-tokens``,
``--temperature``, ``--max-num-seqs``, ``--max-model-len`` (examples/minimal_engine.py:24-55);
``--page-size``, ``--eager`` (benchmark/bench_miniinfer.py:16-26); ``--profile FILE`` stands where the reference
has benchmark/profile_miniinfer.py.  ``--temperature`` and
``--sampler-temp`` are two names of one option.

Without a tokenizer in the model folder, give the prompt as token ids (``--prompt-ids 1,2,3``) or
let ``--prompt-len N`` draw N random ids.  ``--random-weights CONFIG.json`` first writes a model
folder with random weights to ``--model``.
"""
import argparse
import json
import random
import sys
import time


def main(argv=None) -> int:
  p = argparse.ArgumentParser(description="miniinfer_b200: generate from a model folder")
  p.add_argument("--model", required=True, help="local model folder (config.json + *.safetensors)")
  p.add_argument("--prompt", action="append", default=[], help="text prompt (needs tokenizer.json); may repeat")
  p.add_argument("--prompt-ids", action="append", default=[], help="prompt as comma-separated token ids; may repeat")
  p.add_argument("--prompt-len", type=int, default=0, help="draw a random prompt of this many tokens")
  p.add_argument("--max-tokens", type=int, default=64)
  p.add_argument("--temperature", "--sampler-temp", dest="temperature", type=float, default=0.7)
  p.add_argument("--sampler-top-p", "--top-p", dest="top_p", type=float, default=1.0)
  p.add_argument("--sampler-top-k", "--top-k", dest="top_k", type=int, default=0)
  p.add_argument("--ignore-eos", action="store_true")
  p.add_argument("--seed", type=int, default=0)
  p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
  p.add_argument("--device", default="cuda:0")
  p.add_argument("--max-num-seqs", type=int, default=4)
  p.add_argument("--max-model-len", type=int, default=512)
  p.add_argument("--max-num-batched-tokens", type=int, default=2048)
  p.add_argument("--page-size", type=int, default=64)
  p.add_argument("--num-pages", type=int, default=None)
  p.add_argument("--eager", action="store_true", help="no CUDA graphs for decode steps")
  p.add_argument("--profile", metavar="FILE", default=None,
                 help="run the generation under torch.profiler with stage ranges around the phases of a step "
                      "(schedule, describe+launch, wait+update) and write their host times and the kernels' device times to FILE")
  p.add_argument("--random-weights", metavar="CONFIG_JSON", default=None,
                 help="write random weights for this config.json into --model first")
  args = p.parse_args(argv)

  from miniinfer_b200 import LLMEngine, SamplingParams

  if args.random_weights:
    from miniinfer_b200.weights import write_random_model
    with open(args.random_weights, encoding="utf-8") as f:
      write_random_model(json.load(f), args.model, seed=args.seed)

  engine = LLMEngine(args.model, dtype=args.dtype, device=args.device, max_num_seqs=args.max_num_seqs,
                     max_model_len=args.max_model_len, max_num_batched_tokens=args.max_num_batched_tokens,
                     page_size=args.page_size, num_pages=args.num_pages, enforce_eager=args.eager, seed=args.seed)
  prompts = list(args.prompt)
  prompts += [[int(t) for t in s.split(",") if t.strip()] for s in args.prompt_ids]
  if args.prompt_len > 0:
    rng = random.Random(args.seed)
    prompts.append([rng.randrange(engine.model_config.vocab_size) for _ in range(args.prompt_len)])
  if not prompts:
    p.error("give --prompt, --prompt-ids or --prompt-len")
  params = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, top_k=args.top_k,
                          top_p=args.top_p, ignore_eos=args.ignore_eos)
  t0 = time.time()
  with engine:
    if args.profile:
      from miniinfer_b200.utils import profile_to
      with profile_to(args.profile):
        outputs = engine.generate(prompts, params)
    else:
      outputs = engine.generate(prompts, params)
  dt = time.time() - t0
  for prompt, out in zip(prompts, outputs):
    shown = prompt if isinstance(prompt, str) else f"{len(prompt)} token ids"
    print(f"[Prompt]: {shown}")
    print(f"[Response]: {out['text'] if out['text'] is not None else out['token_ids']}")
    print(f"[Token count]: {len(out['token_ids'])}  [finish]: {out['finish_reason']}")
  n = sum(len(o["token_ids"]) for o in outputs)
  print(f"{n} tokens in {dt:.2f} s ({n / dt:.1f} tok/s)")
  return 0


if __name__ == "__main__":
  sys.exit(main())
