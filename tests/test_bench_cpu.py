"""Host-side logic of bench.py that needs no GPU: which parallel layouts the decoder extra times at each GPU count, and that
the reference arm prints a well-formed line on the host cores."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def test_decoder_candidates_cover_pure_and_grouped_tensor_parallelism():
    import bench
    assert [(c["tp"], c["micro_batches"]) for c in bench.decoder_candidates(1)] == [(1, 1), (1, 2), (1, 4)]   # one GPU: whole batch, then groups of sequences
    for world in (2, 4, 8):
        cands = bench.decoder_candidates(world)
        assert [c["micro_batches"] for c in cands if c.get("whole_batch")] == [1, 4] and all(c.get("whole_batch") for c in cands[-2:])   # T1 of the same run, timed last
        cands = cands[:-2]
        assert [c["tp"] for c in cands[:3]] == [world] * 3            # pure tensor parallelism is timed first
        degrees = [c["tp"] for c in cands]
        assert degrees == sorted(degrees, reverse=True) and degrees[-1] == 1 and set(degrees) == {world >> i for i in range(world.bit_length())}
        for c in cands:
            groups = world // c["tp"]
            assert 8 % groups == 0 and (8 // groups) % c["micro_batches"] == 0   # every group gets whole sequences
            assert (c["nccl_max_ctas"] == 0) == (c["sms_left_to_nccl"] == 0)
            assert "fused" not in c                                     # the fused exchange is timed only on request
            assert c["tp"] > 1 or c["micro_batches"] == 1               # replicas have nothing to overlap


def test_fused_candidates_are_added_on_request():
    import bench
    extra = [c for c in bench.decoder_candidates(8, fused=True) if c.get("fused")]
    assert [(c["tp"], c["micro_batches"], c.get("overlap_exchange", False), c.get("pull_exchange", False)) for c in extra if not c.get("dma_exchange") and not c.get("side_scatter")] == [
        (8, 1, False, False), (8, 2, True, False), (8, 1, False, True), (8, 2, True, True), (8, 4, True, True)] + [(8, 2, True, True)] * 5 + [(8, 4, True, True)]
    assert [(c["micro_batches"], c.get("overlap_exchange", False), c["sms_left_to_nccl"]) for c in extra if c.get("dma_exchange")] == [(1, False, 0), (2, True, 0), (4, True, 0)]
    assert [(c["micro_batches"], c.get("overlap_exchange", False), c["sms_left_to_nccl"]) for c in extra if c.get("side_scatter")] == [(1, False, 0), (2, True, 8), (2, True, 16), (2, True, 24)]
    assert all(c["nccl_max_ctas"] == 0 for c in extra)                  # NCCL is not on this path
    assert bench.decoder_candidates(1, fused=True) == bench.decoder_candidates(1)


def test_reference_arm_prints_one_json_line():
    env = dict(os.environ, RANK="0", WORLD_SIZE="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0", "--reference-seconds", "0.2"],
                         capture_output=True, text=True, timeout=240, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] and line["value"] > 0 and line["cpu_baseline"]["kind"] == "port"
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
