"""Submit every ``config.json`` under a directory as a Slurm job and track its status.

    python submit_slurm_jobs.py --inp_dir tmp/sweep --qos normal [--only fail|oom|timeout|pending]
                                [--hf_token ...] [--nb_slurm_array N] [--dry_run]

Each run directory gets a ``status.txt`` that moves through ``init -> pending -> running ->
{completed, fail, oom, timeout}`` (written here and by ``template/base_job.slurm``), a rendered
``job.slurm`` and the job's log; ``--only`` resubmits the runs in a given state. The world size
of a job is ``tp * cp * ep * pp * dp`` (the reference's launcher leaves ``ep`` out,
submit_slurm_jobs.py:83-88). Jobs can be chained with ``--nb_slurm_array`` so that at most that
many run at once (each chain member depends on the previous one finishing).
"""
import argparse
import json
import os
import subprocess
from enum import Enum

GPUS_PER_NODE = 8


class Status(Enum):
    INIT = "init"
    PENDING = "pending"
    RUNNING = "running"
    FAIL = "fail"
    OOM = "oom"
    TIMEOUT = "timeout"
    COMPLETED = "completed"


class Job:
    def __init__(self, root_path: str, qos: str):
        self.root_path = root_path
        self.name = os.path.basename(root_path)
        self.config = os.path.join(root_path, "config.json")
        self.qos = qos
        self.status_path = os.path.join(root_path, "status.txt")
        if not os.path.exists(self.status_path):
            self.set_status(Status.INIT)
        self.status = self.get_status()

    def get_status(self) -> Status:
        raw = open(self.status_path).read().strip()
        return Status(raw) if raw in Status._value2member_map_ else Status.INIT

    def set_status(self, status: Status) -> Status:
        with open(self.status_path, "w") as fh:
            fh.write(status.value)
        self.status = status
        return status

    def world_size(self) -> int:
        d = json.load(open(self.config))["distributed"]
        n = 1
        for k in ("tp_size", "cp_size", "ep_size", "pp_size", "dp_size"):
            n *= int(d.get(k, 1))
        return n


class Scheduler:
    def __init__(self, inp_dir: str, qos: str):
        self.jobs = [Job(root, qos) for root, _, files in sorted(os.walk(inp_dir)) if "config.json" in files]

    def select(self, only: str = None):
        if only is None:
            return [j for j in self.jobs if j.status == Status.INIT]
        return [j for j in self.jobs if j.status.value == only]

    def render(self, job: Job, time_limit: str = "01:00:00") -> str:
        import jinja2
        repo = os.path.dirname(os.path.abspath(__file__))
        tpl = jinja2.Template(open(os.path.join(repo, "template", "base_job.slurm")).read())
        world = job.world_size()
        nodes = max(1, (world + GPUS_PER_NODE - 1) // GPUS_PER_NODE)
        per_node = min(world, GPUS_PER_NODE)
        assert nodes * per_node == world, f"{job.name}: world size {world} does not fill whole nodes"
        text = tpl.render(job_name=f"pico-{job.name}", nodes=nodes, n_proc_per_node=per_node, time_limit=time_limit,
                          root_path=os.path.abspath(job.root_path), qos=job.qos, repo_path=repo,
                          config=os.path.abspath(job.config))
        path = os.path.join(job.root_path, "job.slurm")
        with open(path, "w") as fh:
            fh.write(text)
        return path

    def submit(self, jobs, nb_chains: int = 0, dry_run: bool = False, env=None):
        last_in_chain = {}
        for i, job in enumerate(jobs):
            script = self.render(job)
            cmd = ["sbatch", "--parsable"]
            chain = i % nb_chains if nb_chains > 0 else None
            if chain is not None and chain in last_in_chain:
                cmd.append(f"--dependency=afterany:{last_in_chain[chain]}")
            cmd.append(script)
            if dry_run:
                print(" ".join(cmd))
                continue
            out = subprocess.run(cmd, check=True, capture_output=True, text=True, env=env).stdout.strip()
            job_id = out.split(";")[0]
            if chain is not None:
                last_in_chain[chain] = job_id
            job.set_status(Status.PENDING)
            print(f"submitted {job.name} as {job_id}")

    def summary(self):
        counts = {}
        for j in self.jobs:
            counts[j.status.value] = counts.get(j.status.value, 0) + 1
        return counts


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--inp_dir", type=str, required=True)
    ap.add_argument("--qos", type=str, default="")
    ap.add_argument("--only", type=str, default=None, choices=[s.value for s in Status])
    ap.add_argument("--hf_token", type=str, default=None)
    ap.add_argument("--nb_slurm_array", type=int, default=0)
    ap.add_argument("--dry_run", action="store_true")
    args = ap.parse_args()
    sched = Scheduler(args.inp_dir, args.qos)
    env = dict(os.environ)
    if args.hf_token:
        env["HUGGINGFACE_TOKEN"] = args.hf_token
    todo = sched.select(args.only)
    print(f"{len(sched.jobs)} runs found, {len(todo)} to submit; states: {sched.summary()}")
    sched.submit(todo, args.nb_slurm_array, args.dry_run, env)


if __name__ == "__main__":
    main()
