#!/usr/bin/env python3
"""Stand-in for the `hadoop` command in tests: `fake_hadoop.py fs -mkdir -p | -put -f (- | FILE) | -get | -cat | -ls | -rm -f`.
`hdfs://<anything>/<path>` maps to `$FAKE_HDFS_ROOT/<path>`; every call is appended to `$FAKE_HDFS_ROOT/calls.log`,
so a test can check that the files really went through the command."""
import os
import sys
import time


def local(uri):
    assert uri.startswith("hdfs://"), uri
    rest = uri[len("hdfs://"):]
    return os.path.join(os.environ["FAKE_HDFS_ROOT"], rest.split("/", 1)[1] if "/" in rest else "")


def main():
    args = sys.argv[1:]
    with open(os.path.join(os.environ["FAKE_HDFS_ROOT"], "calls.log"), "a") as log:
        log.write(" ".join(args) + "\n")
    if not args or args[0] != "fs":
        return 2
    op, rest = args[1], [a for a in args[2:] if not (a.startswith("-") and a != "-")]
    if op == "-mkdir":
        os.makedirs(local(rest[0]), exist_ok=True)
    elif op == "-put":
        dst = local(rest[1])
        with open(dst + ".part", "wb") as f:
            if rest[0] == "-":
                f.write(sys.stdin.buffer.read())
            else:
                with open(rest[0], "rb") as src:
                    f.write(src.read())
        os.replace(dst + ".part", dst)
    elif op == "-get":
        with open(local(rest[0]), "rb") as src, open(rest[1], "wb") as f:
            f.write(src.read())
    elif op == "-cat":
        with open(local(rest[0]), "rb") as f:
            sys.stdout.buffer.write(f.read())
    elif op == "-ls":
        d = local(rest[0])
        if not os.path.isdir(d):
            sys.stderr.write(f"ls: `{rest[0]}': No such file or directory\n")
            return 1
        names = sorted(os.listdir(d))
        print(f"Found {len(names)} items")
        for n in names:
            p = os.path.join(d, n)
            kind = "drwxr-xr-x   -" if os.path.isdir(p) else "-rw-r--r--   3"
            stamp = time.strftime("%Y-%m-%d %H:%M", time.localtime(os.path.getmtime(p)))
            print(f"{kind} user supergroup {os.path.getsize(p):>10} {stamp} {rest[0].rstrip('/')}/{n}")
    elif op == "-rm":
        try:
            os.remove(local(rest[0]))
        except FileNotFoundError:
            pass
    else:
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
