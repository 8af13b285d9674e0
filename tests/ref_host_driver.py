"""Child process of tests/ref_host.py: drives `redline.Engine` - the reference's own pybind module
(src/api/pybind.cpp) over whichever kernel library it was linked to - through its public surface only:
Engine(...), add_request, step, has_capacity, stats. Reads one JSON job on stdin, prints one JSON line."""
import json
import sys
import time


def main():
    job = json.loads(sys.stdin.read())
    sys.path.insert(0, job["module_dir"])
    import redline
    t0 = time.perf_counter()
    eng = redline.Engine(job["model_dir"], **job["engine"])
    load_s = time.perf_counter() - t0
    ids, had_capacity = [], []
    for rq in job["requests"]:
        had_capacity.append(bool(eng.has_capacity()))
        ids.append(eng.add_request(rq["prompt"], rq["max_new_tokens"], True, rq.get("forced_tokens")))
    tokens = {i: [] for i in ids}
    reasons = {}
    t0 = time.perf_counter()
    for _ in range(100000):
        for rid, tok, fin, why in eng.step():
            tokens[rid].append(int(tok))
            if fin:
                reasons[rid] = why
        s = eng.stats()
        if s["running"] == 0 and s["waiting"] == 0:
            break
    step_s = time.perf_counter() - t0
    s = eng.stats()
    s["bucket_histogram"] = {str(k): int(v) for k, v in s["bucket_histogram"].items()}
    errors = {}
    try:
        eng.add_request([], 4)
    except Exception as e:   # the binding maps std::invalid_argument to ValueError
        errors["empty_prompt"] = type(e).__name__
    try:
        eng.add_request([10 ** 7], 4)
    except Exception as e:
        errors["token_outside_vocabulary"] = type(e).__name__
    print(json.dumps({"version": redline.__version__, "tokens": [tokens[i] for i in ids],
                      "reasons": [reasons.get(i, "") for i in ids], "had_capacity": had_capacity, "stats": s,
                      "errors": errors, "load_seconds": round(load_s, 2), "step_seconds": round(step_s, 2)}))


if __name__ == "__main__":
    main()
