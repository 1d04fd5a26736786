"""Job launcher (the counterpart of ``tools/launch.py``): starts one worker process per GPU.

    python -m mxnet_b200.parallel.launch -n 8 python train.py --epochs 1
    python -m mxnet_b200.parallel.launch -n 16 -H hosts.txt --launcher ssh python train.py

``local`` starts ``-n`` processes on this machine; ``ssh`` spreads them over the hosts of ``-H`` (one
name per line, ``-n`` divided evenly).  Every worker gets ``RANK``, ``LOCAL_RANK``, ``WORLD_SIZE``,
``MASTER_ADDR``, ``MASTER_PORT`` and, for scripts written against the reference, ``DMLC_ROLE=worker``,
``DMLC_NUM_WORKER``, ``DMLC_WORKER_ID``, ``DMLC_PS_ROOT_URI``, ``DMLC_PS_ROOT_PORT``.  There are no server or
scheduler processes: ranks are peers and rendezvous through rank 0.  The launcher exits with the first
non-zero worker status and stops the remaining workers of the same job (their exact process handles)."""
import argparse
import os
import shlex
import signal
import socket
import subprocess
import sys


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def worker_env(rank, local_rank, world, addr, port, base=None):
    env = dict(base if base is not None else os.environ)
    env.update({'RANK': str(rank), 'LOCAL_RANK': str(local_rank), 'WORLD_SIZE': str(world), 'MASTER_ADDR': addr,
                'MASTER_PORT': str(port), 'DMLC_ROLE': 'worker', 'DMLC_NUM_WORKER': str(world), 'DMLC_NUM_SERVER': '0',
                'DMLC_WORKER_ID': str(rank), 'DMLC_PS_ROOT_URI': addr, 'DMLC_PS_ROOT_PORT': str(port)})
    return env


def launch_local(n, command, addr='127.0.0.1', port=None, env_extra=None):
    port = port or _free_port()
    procs = []
    for r in range(n):
        env = worker_env(r, r, n, addr, port)
        env.update(env_extra or {})
        procs.append(subprocess.Popen(command, env=env))
    return _wait(procs)


def ssh_commands(n, hosts, command, port, env_extra=None):
    """The ssh command lines of an ``n``-worker job over ``hosts`` (pure function: testable without ssh)."""
    per = (n + len(hosts) - 1) // len(hosts)
    addr = hosts[0]
    cmds, rank = [], 0
    for h in hosts:
        for local in range(per):
            if rank >= n:
                break
            env = worker_env(rank, local, n, addr, port, base={})
            env.update(env_extra or {})
            exports = ' '.join('%s=%s' % (k, shlex.quote(v)) for k, v in sorted(env.items()))
            remote = 'cd %s && env %s %s' % (shlex.quote(os.getcwd()), exports, ' '.join(shlex.quote(c) for c in command))
            cmds.append(['ssh', '-o', 'StrictHostKeyChecking=no', h, remote])
            rank += 1
    return cmds


def _wait(procs):
    rc = 0
    try:
        pending = list(procs)
        while pending:
            for p in list(pending):
                code = p.poll()
                if code is None:
                    continue
                pending.remove(p)
                if code != 0 and rc == 0:
                    rc = code
                    for q in pending:           # stop the rest of THIS job: exact handles, no pattern matching
                        q.send_signal(signal.SIGTERM)
            if pending:
                try:
                    pending[0].wait(timeout=0.2)
                except subprocess.TimeoutExpired:
                    pass
    except KeyboardInterrupt:
        for p in procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
        rc = 130
    return rc


def main(argv=None):
    ap = argparse.ArgumentParser(description='Launch a distributed job')
    ap.add_argument('-n', '--num-workers', required=True, type=int)
    ap.add_argument('-s', '--num-servers', type=int, default=0, help='accepted for compatibility; there are no servers')
    ap.add_argument('-H', '--hostfile', type=str)
    ap.add_argument('--launcher', default='local', choices=['local', 'ssh'])
    ap.add_argument('--port', type=int, default=None)
    ap.add_argument('--env', action='append', default=[], help='NAME=VALUE passed to every worker')
    ap.add_argument('command', nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    if not args.command:
        ap.error('no command given')
    extra = dict(e.split('=', 1) for e in args.env)
    if args.launcher == 'local':
        return launch_local(args.num_workers, args.command, port=args.port, env_extra=extra)
    if not args.hostfile:
        ap.error('--launcher ssh needs -H hostfile')
    hosts = [l.strip() for l in open(args.hostfile) if l.strip() and not l.startswith('#')]
    cmds = ssh_commands(args.num_workers, hosts, args.command, args.port or 9091, extra)
    return _wait([subprocess.Popen(c) for c in cmds])


if __name__ == '__main__':
    sys.exit(main())
