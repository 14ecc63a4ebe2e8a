"""Leader/follower engine protocol on CPU (gloo): rank 0 drives, rank 1 replays; both end in the same KV state."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from sllm_b200.engine.distributed import LeaderEngine, follow  # noqa: E402
from sllm_b200.engine.engine import build_engine  # noqa: E402
from sllm_b200.engine.scheduler import EngineLoop, GenRequest  # noqa: E402
from sllm_b200.models import config as MC  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    cfg = MC.tiny_llama()
    cfg.max_context = 128
    pairs = (cfg.rotary_dim or cfg.head_dim) // 2
    cfg.mrope_sections = [pairs // 4, (pairs - pairs // 4) // 2]       # 3-axis rotary sections (multimodal prompts)
    eng = build_engine(cfg, "cpu", seed=1, num_pages=64, max_batch=4, use_cuda_graphs=False)
    if rank == 0:
        lead = LeaderEngine(eng)
        want = build_engine(cfg, "cpu", seed=1, num_pages=64, max_batch=4, use_cuda_graphs=False).generate([[1, 2, 3, 4], [9, 8, 7]], 6)
        assert lead.generate([[1, 2, 3, 4], [9, 8, 7]], 6) == want
        # the continuous-batching loop on top of the mirrored engine
        import time
        loop = EngineLoop(lead)
        toks, done = [], []
        loop.submit(GenRequest(prompt=[1, 2, 3, 4], max_new_tokens=6, on_token=lambda t, s: toks.append(t) or True, on_done=done.append))
        for _ in range(2000):
            if done:
                break
            time.sleep(0.005)
        loop.shutdown(2.0)
        assert done == ["length"] and toks == want[0]
        # a multimodal prompt: spliced input rows and 3-axis positions are mirrored with the command
        mm_tokens, d = [5, 6, 7, 8, 9, 10], cfg.d_model
        g = torch.Generator().manual_seed(7)
        embeds = (torch.randn(len(mm_tokens), d, generator=g) * 0.05).to(eng.model.w.embed.dtype)
        pos3 = torch.tensor([[0, 1, 1, 1, 2, 3], [0, 1, 1, 2, 2, 3], [0, 1, 2, 1, 2, 3]], dtype=torch.int32)
        ref_eng = build_engine(cfg, "cpu", seed=1, num_pages=64, max_batch=4, use_cuda_graphs=False)
        rs = ref_eng.new_sequence(mm_tokens)
        want_first = ref_eng.prefill([rs], embeds=embeds, rope_pos3=pos3, one_chunk=True)
        rs.tokens.append(want_first[0])
        want_next = ref_eng.decode([rs])
        s = lead.new_sequence(mm_tokens)
        first = lead.prefill([s], embeds=embeds, rope_pos3=pos3, one_chunk=True)
        s.tokens.append(first[0])
        nxt = lead.decode([s])
        assert (first, nxt) == (want_first, want_next), (first, nxt, want_first, want_next)
        mm_delta = s.rope_delta
        lead.free_sequence(s)
        ref_eng.free_sequence(rs)
        # hidden rows for the embeddings endpoint: mirrored too
        assert torch.equal(lead.embed_hidden([3, 4, 5, 6, 7]), ref_eng.embed_hidden([3, 4, 5, 6, 7]))
        lead.stop_followers()
    else:
        handled = follow(eng)
        assert handled > 10
        mm_delta = None
    st = eng.cache.pool.stats()
    assert st["sequences"] == 0 and st["free"] == st["pages"], st
    gathered = [None, None]
    dist.all_gather_object(gathered, st["high_water"])
    assert gathered[0] == gathered[1], gathered          # both ranks allocated the same pages
    dist.barrier()
    if rank == 0:
        print("DIST_ENGINE_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
