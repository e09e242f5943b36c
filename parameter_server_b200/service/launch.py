"""Process launchers of the service layer.

    python -m parameter_server_b200.service.launch master [--port P] [--state-file F]   # prints the address, serves until killed
    python -m parameter_server_b200.service.launch pserver --master 127.0.0.1:PORT [--restore] [--image-dir DIR]
        [--restore-wait S] [--report-interval S] [--sync-master ADDR] [--metrics-port P] [--hadoop-bin PATH] [--log-level L]

A ``pserver`` registers at the master, serves its c2s / s2s ports and exits when a client sends EXIT
(``Controller.shutdown_node``). With ``--restore`` it first takes over the shards of a dead node
(``Server.restore_storages``), the restore mode of the reference's pserver binary
(pico-ps/service/Service.cpp:237-313).
"""
from __future__ import annotations

import argparse
import sys
import time

from . import Master, Server, ServerConfig, TableSyncer, set_log_level


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="parameter_server_b200.service.launch")
    sub = ap.add_subparsers(dest="role", required=True)
    m = sub.add_parser("master")
    m.add_argument("--threads", type=int, default=4)
    m.add_argument("--port", type=int, default=0, help="fixed port (needed to find a restarted master again)")
    m.add_argument("--state-file", default="", help="durable state: a restarted master carries on from it")
    p = sub.add_parser("pserver")
    p.add_argument("--master", required=True)
    p.add_argument("--restore", action="store_true")
    p.add_argument("--restore-pauses-writes", action="store_true",
                   help="close a table to writes while it is copied from the live replicas (the new replica is exact)")
    p.add_argument("--image-dir", default="", help="persistent table images: written on a planned shutdown, opened in restore mode")
    p.add_argument("--c2s-threads", type=int, default=4)
    p.add_argument("--s2s-threads", type=int, default=4)
    p.add_argument("--restore-wait", type=int, default=-1, help="seconds a restore-mode server keeps looking for a dead node")
    p.add_argument("--report-interval", type=int, default=-1, help="seconds between status lines (also the memory monitor's interval)")
    p.add_argument("--sync-master", default="", help="master of the cluster that holds the follower tables (starts the sync thread)")
    p.add_argument("--metrics-port", type=int, default=-1, help="Prometheus endpoint (0 = any free port)")
    p.add_argument("--hadoop-bin", default="", help="command behind hdfs:// dump paths")
    p.add_argument("--log-level", default="", help="debug | info | warning | error | off")
    a = ap.parse_args(argv)
    if a.role == "pserver" and a.log_level:
        set_log_level(a.log_level)
    if a.role == "master":
        master = Master(a.threads, a.port, a.state_file)
        print(master.address(), flush=True)
        try:
            while True:
                time.sleep(3600)
        except KeyboardInterrupt:
            master.stop()
        return 0
    cfg = ServerConfig()
    cfg.c2s_thread_num, cfg.s2s_thread_num = a.c2s_threads, a.s2s_threads
    cfg.local_image_dir = a.image_dir
    cfg.restore_wait_timeout_s, cfg.report_interval_s, cfg.hadoop_bin = a.restore_wait, a.report_interval, a.hadoop_bin
    cfg.restore_pauses_writes = a.restore_pauses_writes
    server = Server(a.master, cfg)
    print(f"pserver node_id={server.node_id()} c2s={server.c2s_address()} s2s={server.s2s_address()}", flush=True)
    httpd = None
    if a.metrics_port >= 0:
        from .metrics import serve_metrics
        httpd, port = serve_metrics(server, a.metrics_port)
        print(f"metrics port={port}", flush=True)
    syncer = TableSyncer(server, a.sync_master) if a.sync_master else None
    if a.restore:
        st, n = server.restore_storages()
        print(f"restore: {st} ({n} tables)", flush=True)
        if not st.ok():
            return 1
    try:
        while not server.exited():
            time.sleep(0.05)
    except KeyboardInterrupt:
        pass
    if httpd is not None:
        httpd.shutdown()
    if syncer is not None:
        syncer.wait_idle(5000)
        syncer.stop()
    if a.image_dir:
        st, n = server.save_local_images()
        print(f"images: {st} ({n} tables)", flush=True)
    server.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
