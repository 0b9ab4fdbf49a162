"""The N>1 plumbing of the benchmark (barrier, max over ranks, whole-job throughput, rank-0-only
reporting) with two gloo ranks on the CPU."""
import json
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(script, world=2, extra_args=()):
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), PYTHONPATH=ROOT)
        procs.append(subprocess.Popen([sys.executable, "-c", script, *extra_args], env=env, cwd=ROOT,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=240)
        assert p.returncode == 0, err[-2000:]
        outs.append(out)
    return outs


def test_max_over_ranks_and_job_throughput_world_2():
    script = textwrap.dedent("""
        import json, time
        from better_benchmark_b200.replicas import ReplicaGroup
        g = ReplicaGroup(backend="gloo")
        g.barrier()
        mine = 0.010 * (g.rank + 1)            # rank 0: 10 ms, rank 1: 20 ms
        slowest = g.max_over_ranks(mine)
        thr = g.job_throughput(1000.0, mine)   # 1000 units per rank
        g.barrier()
        print(json.dumps({"rank": g.rank, "world": g.world, "slowest": slowest, "thr": thr,
                          "reporter": g.is_reporter()}))
        g.close()
    """)
    outs = [json.loads(o.strip().splitlines()[-1]) for o in _launch(script)]
    assert sorted(o["rank"] for o in outs) == [0, 1]
    for o in outs:
        assert o["world"] == 2
        assert abs(o["slowest"] - 0.020) < 1e-12, "every rank must see the slowest rank's time"
        assert abs(o["thr"] - 2000.0 / 0.020) < 1e-6, "whole-job units over the slowest time"
    assert [o["reporter"] for o in sorted(outs, key=lambda o: o["rank"])] == [True, False]


def test_single_process_group_is_local():
    from better_benchmark_b200.replicas import ReplicaGroup
    env = {k: os.environ.pop(k) for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE") if k in os.environ}
    try:
        g = ReplicaGroup()
        g.barrier()
        assert g.world == 1 and g.max_over_ranks(3.5) == 3.5 and g.job_throughput(10, 2) == 5.0
        g.close()
    finally:
        os.environ.update(env)


def test_reference_arm_reports_on_rank_0_only():
    """bench.py --impl reference under a 2-rank launch: rank 0 prints the line, rank 1 exits 0 silent."""
    script = textwrap.dedent("""
        import sys
        sys.argv = ["bench.py", "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "3",
                    "--workload", "c1_row_mean"]
        import bench
        sys.exit(bench.main())
    """)
    outs = _launch(script)
    lines = [o.strip() for o in outs]
    assert sum(1 for l in lines if l) == 1, "exactly one rank reports"
    line = json.loads([l for l in lines if l][0].splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["unit"] == "GB/s"
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["config"]["workload"] == "c1_row_mean" and line["value"] > 0
