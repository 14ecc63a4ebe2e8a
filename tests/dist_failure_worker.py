"""Failure paths of the leader/follower protocol on CPU (gloo), made on the host: a follower that raises in the
middle of a step, and a leader that goes away.  SLLM_TEST_FAIL selects the case."""
import datetime
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from sllm_b200.engine.distributed import FollowerFailed, LeaderEngine, LeaderLost, follow  # noqa: E402
from sllm_b200.engine.engine import build_engine  # noqa: E402
from sllm_b200.models import config as MC  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    case = os.environ["SLLM_TEST_FAIL"]
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
    cfg = MC.tiny_llama()
    cfg.max_context = 128
    eng = build_engine(cfg, "cpu", seed=1, num_pages=64, max_batch=4, use_cuda_graphs=False)
    if case == "follower_raises":
        if rank == 0:
            lead = LeaderEngine(eng)
            s = lead.new_sequence([1, 2, 3, 4])
            s.tokens.append(lead.prefill([s])[0])
            try:
                for _ in range(50):
                    s.tokens.append(lead.decode([s])[0])
                print("NO_FAILURE_SEEN", flush=True)
            except FollowerFailed as exc:
                # the leader's own engine is intact: it finished every step it launched
                assert "injected decode failure" in str(exc) or "command channel failed" in str(exc), str(exc)
                assert eng.cache.pool.length(s.seq_id) == len(s.tokens) - 1
                print("LEADER_SAW_FOLLOWER_FAILURE", flush=True)
        else:
            calls = {"n": 0}
            real = eng.decode

            def flaky(seqs, sample=True):
                calls["n"] += 1
                if calls["n"] == 3:
                    raise RuntimeError("injected decode failure")
                return real(seqs, sample)

            eng.decode = flaky
            try:
                follow(eng)
            except RuntimeError as exc:
                assert "injected decode failure" in str(exc)
                print("FOLLOWER_REPORTED_AND_LEFT", flush=True)
    elif case == "leader_stops":
        if rank == 0:
            lead = LeaderEngine(eng)
            s = lead.new_sequence([5, 6, 7])
            s.tokens.append(lead.prefill([s])[0])
            print("LEADER_EXITS_WITHOUT_STOP", flush=True)     # no stop command: the follower must notice by itself
        else:
            try:
                follow(eng)
                print("FOLLOWER_RETURNED_NORMALLY", flush=True)
            except LeaderLost:
                print("FOLLOWER_SAW_LEADER_LOSS", flush=True)
    sys.stdout.flush()
    os._exit(0)      # the peer is gone: skip the collective teardown of the process group


if __name__ == "__main__":
    main()
