"""Command-line surface of the bound-propagation path: `python -m ny_b200 beta-crown MODEL -p PROPERTY` and
`python -m ny_b200 verify MODEL -p PROPERTY [--method ibp|crown]`, with the reference's result block and exit codes
(README.md:82-122 of the reference: 0 proved, 1 falsified, 2 unknown, 3 timeout, 4 invalid invocation or
operational error; `--allow-unknown` maps unknown to 0).  Models: .nnet, .onnx (sequential ReLU subset);
properties: the VNN-LIB subset of ny_b200.formats.  Certificates, presets and the other subcommands are not part
of this path."""
from __future__ import annotations

import argparse
import sys

import numpy as np

EXIT = {"verified": 0, "violated": 1, "unknown": 2, "timeout": 3}


def _load_model(path):
    from . import formats, onnx_reader

    if path.endswith(".nnet"):
        return formats.parse_nnet(open(path).read()).to_network()
    if path.endswith(".onnx"):
        return onnx_reader.parse_onnx(open(path, "rb").read())[0]
    raise ValueError(f"unsupported model format: {path}")


def _report(res, prop):
    print("--- Result ---")
    print(f"Status: {res.status.upper()}")
    if res.status == "violated":
        print(f"Counterexample input: {np.array2string(np.asarray(res.counterexample), separator=', ')}")
        print(f"Counterexample output: {np.array2string(np.asarray(res.output), separator=', ')}")
    elif res.root_lower is not None:
        print(f"Root lower bounds of the refutation rows: {np.array2string(res.root_lower, separator=', ')}")
    print(f"Domains bounded: {res.domains_bounded}, rounds: {res.rounds}, open: {res.open_domains}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ny_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("beta-crown", "verify"):
        p = sub.add_parser(name)
        p.add_argument("model")
        p.add_argument("-p", "--property", required=True)
        p.add_argument("--timeout", type=float, default=None, help="seconds")
        p.add_argument("--device", type=int, default=0)
        p.add_argument("--allow-unknown", action="store_true")
        if name == "beta-crown":
            p.add_argument("--batch-size", type=int, default=1024)
            p.add_argument("--max-domains", type=int, default=100_000)
            p.add_argument("--beta-iterations", type=int, default=20)
            p.add_argument("--branching", choices=("width", "intercept", "babsr", "fsb"), default="intercept")
            p.add_argument("--input-split", action="store_true", help="branch on input dimensions instead of ReLUs")
            p.add_argument("--domain-batch-metrics-jsonl", default=None)
            p.add_argument("--resident", action="store_true",
                           help="keep the open domain set on the device (one call per round); width / intercept / babsr "
                                "branching, split histories up to --max-depth")
            p.add_argument("--max-depth", type=int, default=128, help="--resident: longest split history")
            p.add_argument("--checkpoint", default=None)
            p.add_argument("--resume", default=None)
        else:
            p.add_argument("--method", choices=("ibp", "crown"), default="crown")
    try:
        args = ap.parse_args(argv)
    except SystemExit as e:
        return 4 if e.code not in (0, None) else 0
    try:
        from . import B200Engine, bab, formats

        net = _load_model(args.model)
        prop = formats.parse_vnnlib(open(args.property).read(), int(net.dims[0]), int(net.dims[-1]))
        eng = B200Engine(args.device)
        nid = eng.register_network(net)
        if args.cmd == "beta-crown":
            if args.input_split:
                res = bab.verify_input_split(eng, nid, net, prop, batch=args.batch_size, max_domains=args.max_domains,
                                             timeout_s=args.timeout)
            else:
                kind = {"width": 0, "intercept": 1, "babsr": 2, "fsb": 3}[args.branching]
                if args.resident:
                    if kind == 3 or args.domain_batch_metrics_jsonl:
                        raise ValueError("--resident supports width, intercept and babsr branching and writes no metrics file")
                    res = bab.verify_resident(eng, nid, net, prop, batch=args.batch_size, max_domains=args.max_domains,
                                              max_rounds=max(1, args.max_depth - 2), optimize_iterations=args.beta_iterations,
                                              branching=kind, timeout_s=args.timeout, checkpoint=args.checkpoint, resume=args.resume,
                                              refinement="verdict")   # a verdict is what this command reports
                else:
                    res = bab.verify(eng, nid, net, prop, batch=args.batch_size, max_domains=args.max_domains, max_rounds=1 << 30,
                                     optimize_iterations=args.beta_iterations, branching=kind, timeout_s=args.timeout,
                                     metrics_jsonl=args.domain_batch_metrics_jsonl, checkpoint=args.checkpoint, resume=args.resume,
                                     refinement="verdict")
        else:
            res = bab.verify_root(eng, nid, net, prop, method=args.method)
        _report(res, prop)
        eng.close()
    except Exception as e:  # operational error: the reference's exit code 4
        print(f"error: {e}", file=sys.stderr)
        return 4
    code = EXIT[res.status]
    return 0 if (code == 2 and args.allow_unknown) else code


if __name__ == "__main__":
    sys.exit(main())
