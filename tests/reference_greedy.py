"""Run by tests/test_gpu_reference_anchor.py in a process of its own: izmttk/ullm itself, unmodified, from
baseline/_ref, through its public API (`ullm.LLM.generate`, ullm/llm.py:76-117), generates greedy tokens
(top_k=1) for the prompts of a JSON file and prints one line `RESULT <json>` with the token strings it
streamed.  Nothing of this repository's engine is imported here.

    python tests/reference_greedy.py MODEL_DIR PROMPTS.json NEW_TOKENS
"""

import asyncio
import json
import os
import sys


def main() -> int:
    model, prompts_file, n_new = sys.argv[1], sys.argv[2], int(sys.argv[3])
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "baseline", "_ref"))
    with open(prompts_file) as f:
        prompts = json.load(f)
    # the reference logs to standard output, from its child processes too: keep descriptor 1 for the result line
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    from ullm import LLM, EngineConfig, SamplingParams  # the reference's public API

    out: list[list[str]] = [[] for _ in prompts]

    async def run():
        llm = LLM(EngineConfig(model=model, gpu_memory_utilization=0.5, max_bs=8, tp_size=1, pp_size=1,
                               nccl_port=29547, device_ids=[0], context_len=512))
        # one request after the other: the reference's default scheduling raises on a prefill step that holds
        # several new requests (ullm/core/input_batch.py:185)
        for i, p in enumerate(prompts):
            sp = SamplingParams(temperature=1.0, top_k=1, ignore_eos=True, max_new_tokens=n_new)
            async for o in llm.generate(p, sp):
                out[i].append(o.token_str)
        await llm.shutdown()

    asyncio.run(run())
    sys.stdout.flush()
    os.dup2(saved, 1)
    os.write(1, ("RESULT " + json.dumps(out) + "\n").encode())
    return 0


if __name__ == "__main__":
    sys.exit(main())
