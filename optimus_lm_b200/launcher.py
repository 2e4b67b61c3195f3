"""Job launcher: one process per GPU on one or many nodes, with an optional node health screen.

The reference starts jobs with ``mpiexec`` over a PBS node file (launch_dist.sh:10-70) and, in its
advanced launcher, first drops nodes that do not answer a ping ("hard" failures) and nodes that an
earlier run of the same job reported for producing non-finite losses ("soft" failures, listed in
``launch_info/<job>/failed_soft_nodes.txt`` by the training driver), then launches on the first
``num_nodes`` healthy ones (launch_dist_advanced.sh:52-131).

Here every node runs ``python -m torch.distributed.run`` (one worker per GPU, NCCL rendezvous on
the first selected node).  One node: the launcher execs it directly.  Several nodes: one agent per
node is started through ``srun`` (inside a SLURM allocation) or ``ssh``.  The health screen is the
same two lists; the probe is a function argument so that tests can inject failures on the host.

    python -m optimus_lm_b200.launcher --gpus_per_node 8 --num_nodes 4 --hostfile nodes.txt --health_check \
        -- dist_train.py --model_choice ... --expert_parallelism 8 --data_parallelism 4
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys
from typing import Callable, Dict, List, Optional, Sequence, Tuple


def read_hostfile(path: str) -> List[str]:
    """Node names, one per line; ``name slots=8`` style suffixes and duplicate lines are dropped."""
    nodes: List[str] = []
    with open(path) as fh:
        for line in fh:
            tok = line.split()
            if tok and not tok[0].startswith("#") and tok[0] not in nodes:
                nodes.append(tok[0])
    return nodes


def ping_probe(node: str) -> bool:
    try:
        return subprocess.run(["ping", "-c", "1", "-W", "1", node], stdout=subprocess.DEVNULL,
                              stderr=subprocess.DEVNULL, timeout=5).returncode == 0
    except (OSError, subprocess.TimeoutExpired):
        return False


def job_id(environ=None) -> str:
    environ = os.environ if environ is None else environ
    return str(environ.get("PBS_JOBID", environ.get("SLURM_JOB_ID", "0"))).split(".")[0]


def launch_info_dir(environ=None) -> str:
    environ = os.environ if environ is None else environ
    return os.path.join(environ.get("OPTIMUS_LAUNCH_INFO_DIR", "launch_info"), job_id(environ))


def read_soft_failures(info_dir: str) -> List[str]:
    path = os.path.join(info_dir, "failed_soft_nodes.txt")
    if not os.path.isfile(path):
        return []
    with open(path) as fh:
        return [ln.strip() for ln in fh if ln.strip()]


def select_nodes(nodes: Sequence[str], num_nodes: int, *, probe: Callable[[str], bool] = ping_probe,
                 soft_failed: Sequence[str] = (), log=print) -> List[str]:
    """First ``num_nodes`` nodes that answer the probe and are not listed as soft-failed.  Raises
    ``RuntimeError`` when too few are left."""
    hard = [n for n in nodes if not probe(n)]
    soft = [n for n in nodes if n in set(soft_failed)]
    good = [n for n in nodes if n not in hard and n not in soft]
    log(f"Number of allocated nodes   : {len(nodes)}")
    log(f"Number of hard failed nodes : {len(hard)}")
    log(f"Number of soft failed nodes : {len(soft)}")
    log(f"Number of good nodes        : {len(good)}")
    log(f"Number of requested nodes   : {num_nodes}")
    log(f"Failed hard nodes : {' '.join(hard)}")
    log(f"Failed soft nodes : {' '.join(soft)}")
    if len(good) < num_nodes:
        raise RuntimeError(f"Not enough good nodes available. Required: {num_nodes}, Available: {len(good)}")
    return good[:num_nodes]


def gpu_health_report(query: Optional[Callable[[], str]] = None) -> List[str]:
    """Read-only screen of this node's GPUs: uncorrected ECC errors, active hardware slowdown.
    Returns human-readable findings (empty = healthy).  Nothing on the GPU is changed."""
    if query is None:
        def query():
            return subprocess.run(
                ["nvidia-smi", "--query-gpu=index,ecc.errors.uncorrected.volatile.total,"
                 "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown",
                 "--format=csv,noheader"], capture_output=True, text=True, timeout=30).stdout
    findings = []
    try:
        out = query()
    except (OSError, subprocess.TimeoutExpired) as e:
        return [f"nvidia-smi could not be run: {e}"]
    for line in out.strip().splitlines():
        f = [t.strip() for t in line.split(",")]
        if len(f) < 4:
            continue
        idx, ecc, hw, therm = f[:4]
        if ecc.isdigit() and int(ecc) > 0:
            findings.append(f"GPU {idx}: {ecc} uncorrected ECC errors")
        if hw.lower() == "active" or therm.lower() == "active":
            findings.append(f"GPU {idx}: hardware slowdown active")
    return findings


def torchrun_command(script_and_args: Sequence[str], gpus_per_node: int, num_nodes: int, node_rank: int,
                     master_addr: str, master_port: int) -> List[str]:
    return [sys.executable, "-m", "torch.distributed.run", f"--nnodes={num_nodes}",
            f"--nproc-per-node={gpus_per_node}", f"--node-rank={node_rank}", "--master-addr", master_addr,
            "--master-port", str(master_port)] + list(script_and_args)


def node_commands(nodes: Sequence[str], script_and_args: Sequence[str], gpus_per_node: int, master_port: int,
                  transport: str, cwd: str, forward_env: Sequence[str] = ()) -> List[List[str]]:
    """One command per node.  ``transport``: ``local`` (single node), ``ssh`` or ``srun``."""
    if len(nodes) == 1 and transport == "local":
        return [torchrun_command(script_and_args, gpus_per_node, 1, 0, "127.0.0.1", master_port)]
    master = nodes[0]
    cmds = []
    for i, node in enumerate(nodes):
        run = torchrun_command(script_and_args, gpus_per_node, len(nodes), i, master, master_port)
        exports = " ".join(f"{k}={shlex.quote(os.environ[k])}" for k in forward_env if k in os.environ)
        remote = f"cd {shlex.quote(cwd)} && {exports} " + " ".join(shlex.quote(c) for c in run)
        if transport == "srun":
            cmds.append(["srun", "--nodes=1", "--ntasks=1", f"--nodelist={node}", "bash", "-lc", remote])
        else:
            cmds.append(["ssh", "-o", "BatchMode=yes", node, remote])
    return cmds


FORWARDED_ENV = ("PBS_JOBID", "SLURM_JOB_ID", "OPTIMUS_LAUNCH_INFO_DIR", "NCCL_DEBUG", "NCCL_NVLS_ENABLE",
                 "NCCL_IB_HCA", "NCCL_SOCKET_IFNAME", "OLB_DISABLE_KERNELS", "OLB_ATTENTION", "PYTHONPATH")


def main(argv: Optional[Sequence[str]] = None, *, probe: Callable[[str], bool] = ping_probe,
         spawn: Callable[[List[str]], "subprocess.Popen"] = None) -> int:
    p = argparse.ArgumentParser(description="Launch one process per GPU on one or more nodes")
    p.add_argument("--gpus_per_node", type=int, default=8)
    p.add_argument("--num_nodes", type=int, default=1)
    p.add_argument("--hostfile", type=str, default=os.environ.get("HOSTFILE_PATH", os.environ.get("PBS_NODEFILE", "")))
    p.add_argument("--health_check", action="store_true", help="drop unreachable and soft-failed nodes first")
    p.add_argument("--master_port", type=int, default=29500)
    p.add_argument("--transport", choices=["auto", "local", "ssh", "srun"], default="auto")
    p.add_argument("--dry_run", action="store_true")
    p.add_argument("command", nargs=argparse.REMAINDER, help="-- script.py args...")
    a = p.parse_args(argv)
    cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
    if not cmd:
        p.error("no command given after --")
    spawn = spawn or (lambda c: subprocess.Popen(c))

    if a.num_nodes == 1 and not a.hostfile:
        nodes, transport = ["127.0.0.1"], "local"
    else:
        if not a.hostfile:
            p.error("--hostfile (or HOSTFILE_PATH / PBS_NODEFILE) is needed for more than one node")
        nodes = read_hostfile(a.hostfile)
        transport = a.transport
        if transport == "auto":
            transport = "srun" if "SLURM_JOB_ID" in os.environ else ("local" if a.num_nodes == 1 else "ssh")
        info = launch_info_dir()
        if a.health_check:
            try:
                nodes = select_nodes(nodes, a.num_nodes, probe=probe, soft_failed=read_soft_failures(info))
            except RuntimeError as e:
                print(f"Error: {e}")
                return 1
            os.makedirs(info, exist_ok=True)
            with open(os.path.join(info, "hostfile"), "w") as fh:
                fh.write("\n".join(nodes) + "\n")
            print(f"Hostfile path  : {os.path.join(info, 'hostfile')}")
        else:
            if len(nodes) < a.num_nodes:
                print(f"Error: hostfile lists {len(nodes)} nodes, {a.num_nodes} requested")
                return 1
            nodes = nodes[:a.num_nodes]
        print(f"Master address : {nodes[0]}")
    if a.health_check and transport == "local":
        for finding in gpu_health_report():
            print(f"Warning: {finding}")

    cmds = node_commands(nodes, cmd, a.gpus_per_node, a.master_port, transport, os.getcwd(), FORWARDED_ENV)
    for c in cmds:
        print(" ".join(shlex.quote(t) for t in c), flush=True)
    if a.dry_run:
        return 0
    procs = [spawn(c) for c in cmds]
    rc = 0
    for pr in procs:
        r = pr.wait()
        rc = rc or r
    return rc


if __name__ == "__main__":
    sys.exit(main())
