"""KV-range sharding over real GPUs, both forms of the exchange -- NCCL all-gather of packed
partials + merge, and the decode kernels' own peer stores + flags -- against the oracle, and the
failure case of the second form: a rank that is not asked to store.  Needs at least two GPUs
(skipped otherwise); ranks are child processes of torch.distributed.run, NVLS off."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]

WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200 import sharding
from single_gpu_inference_lab_b200.workloads import make_inputs
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
w = make_inputs("llama3-8b-long-b4", seed=0, batch=3, shrink=1 / 32)
lens = w.seq_lens.clone(); lens[1] = 700; lens[2] = 2049; w.seq_lens = lens
ref = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
local = sharding.shard_kv_range(w, rank, world).to("cuda")
out = sharding.kv_range_decode(local, split_size=512)
torch.cuda.synchronize()
err = (out.float().cpu() - ref.float()).abs()
ok = bool((err <= 2e-3 + 1e-2 * ref.float().abs()).all())
# sequence sharding: this rank's sequences alone, no collective
w2 = make_inputs("qwen2.5-7b-b256", seed=1, batch=24, shrink=0.1)
mine, rows = sharding.shard_sequences(w2, rank, world)
g = mine.to("cuda")
from single_gpu_inference_lab_b200 import l20_paged_split_kv as m
o2 = m.l20_paged_split_kv_attention_fp8(g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens,
        k_scale=g.k_scale, v_scale=g.v_scale, max_seq_len=mine.max_seq_len, split_size=128)
ref2 = oracle.reference(w2.query, w2.key_cache, w2.value_cache, w2.block_table.long(), w2.seq_lens, w2.k_scale, w2.v_scale)[rows]
err2 = (o2.float().cpu() - ref2.float()).abs()
ok2 = bool((err2 <= 2e-3 + 1e-2 * ref2.float().abs()).all())
print(f"RANK{{rank}} kv_range_ok={{ok}} max_abs={{err.max().item():.2e}} seq_shard_ok={{ok2}} max_abs={{err2.max().item():.2e}}", flush=True)
dist.destroy_process_group()
sys.exit(0 if ok and ok2 else 1)
"""


@pytest.mark.timeout(600)
def test_kv_range_and_sequence_sharding_on_two_gpus(tmp_path, built_libs):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
        capture_output=True, text=True, env=env, timeout=500,
    )
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "RANK0 kv_range_ok=True" in proc.stdout and "RANK1 kv_range_ok=True" in proc.stdout


EXCHANGE_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200 import cabi, sharding
from single_gpu_inference_lab_b200 import l20_paged_split_kv as m
from single_gpu_inference_lab_b200.workloads import make_inputs
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
torch.cuda.set_device(dev)
dist.init_process_group("nccl")
w = make_inputs("llama3-8b-long-b4", seed=0, batch=3, shrink=1 / 32)
lens = w.seq_lens.clone(); lens[1] = 700; lens[2] = 1; w.seq_lens = lens
ref = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
local = sharding.shard_kv_range(w, rank, world).to(dev)
split = 256
ws = m.allocate_l20_paged_split_kv_workspace(local.query, max(local.max_seq_len, 1), split_size=split)
plan = cabi.plan_decode(local.query, local.key_cache, local.value_cache, local.block_table, local.seq_lens,
                        max_seq_len=local.max_seq_len, split_size=split, workspace=ws)
x = sharding.KvRangeExchange.create(*w.query.shape, dev)
# first launches load the kernels; the ranks then start the exchange steps together
warm = torch.empty_like(local.query)
cabi.paged_decode_fp8_e4m3_split_out(local.query, local.key_cache, local.value_cache, local.block_table, local.seq_lens,
    k_scale=local.k_scale, v_scale=local.v_scale, max_seq_len=local.max_seq_len, split_size=split, workspace=ws, output=warm)
torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()

def gate(out):
    err = (out.float().cpu() - ref.float()).abs()
    return bool((err <= 2e-3 + 1e-2 * ref.float().abs()).all()), err.max().item()

ok, worst = True, 0.0
for step in range(6):
    out = sharding.kv_range_decode_exchange(local, x, split_size=split, workspace=ws, plan=plan if step % 2 else None,
                                            flags=32 if step >= 3 else 0)
    torch.cuda.synchronize()
    good, e = gate(out)
    ok, worst = ok and good and cabi.device_status() == 0, max(worst, e)

# the failure: rank 1 is not asked to store in this step, so its flag arrives nowhere
torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
cabi.set_wait_limit_ns(50_000_000)
out = torch.full_like(local.query, 7.0)
if rank != 1:
    x.decode(local, split_size=split, workspace=ws)
x.merge(out)
status = cabi.device_status()
untouched = bool((out == 7.0).all())
cabi.set_wait_limit_ns(200_000_000)
torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()

after = True
for step in range(3):
    out = sharding.kv_range_decode_exchange(local, x, split_size=split, workspace=ws)
    torch.cuda.synchronize()
    good, e = gate(out)
    after = after and good and cabi.device_status() == 0
print(f"RANK{{rank}} exchange_ok={{ok}} max_abs={{worst:.2e}} missing_status={{status}} untouched={{untouched}} after_ok={{after}}", flush=True)
torch.cuda.synchronize(); dist.barrier()
x.close()
dist.destroy_process_group()
sys.exit(0 if ok and after and status == 4 and untouched else 1)
"""


@pytest.mark.timeout(600)
def test_in_kernel_exchange_on_two_gpus_and_a_rank_that_does_not_publish(tmp_path, built_libs):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "exchange_worker.py"
    script.write_text(EXCHANGE_WORKER.format(root=str(ROOT)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29613", str(script)],
        capture_output=True, text=True, env=env, timeout=500,
    )
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    for r in (0, 1):
        assert f"RANK{r} exchange_ok=True" in proc.stdout, proc.stdout[-2000:]
        assert f"missing_status=4 untouched=True after_ok=True" in proc.stdout
