"""Extract the golden vectors of the reference's own Python tests into JSON.

Run in a checkout that has the reference mounted:
    python tests/golden/make_golden.py <path of the reference checkout>
It reads ``tests/py/test_hist_logregression.py`` and
``tests/py/test_sklearn_classification.py`` as text (nothing is executed), pulls
the expected prediction vectors and the expected model JSON out of the
``run_regression(...)`` calls with ``ast`` and writes ``iris_hist_golden.json``
beside this script.  The iris inputs themselves are not stored: the tests load
them from scikit-learn at run time, exactly like the reference tests do.
"""
import ast
import json
import os
import sys


def _lit(node):
    return ast.literal_eval(node)


def extract_logreg(path):
    tree = ast.parse(open(path).read())
    cases = {}
    for fn in [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name.startswith("test_")]:
        for call in ast.walk(fn):
            if isinstance(call, ast.Call) and getattr(call.func, "id", "") == "run_regression":
                depth = _lit(call.args[0])
                preds = _lit(call.args[1])
                model = json.loads(_lit(call.args[2].args[0]))
                trees = _lit(call.args[3]) if len(call.args) > 3 else 1
                cases[fn.name] = {"max_depth": depth, "trees": trees, "predictions": preds,
                                  "model": model,
                                  "source": "tests/py/test_hist_logregression.py:" + str(fn.lineno)}
    return cases


def extract_sklearn(path):
    tree = ast.parse(open(path).read())
    for fn in [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "test_single_tree"]:
        return {"predictions": _lit(fn.args.defaults[-1]),
                "source": "tests/py/test_sklearn_classification.py:" + str(fn.lineno)}


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REF", "")
    if not os.path.isdir(os.path.join(ref, "tests", "py")):
        raise SystemExit("usage: make_golden.py /path/to/the/reference/tree  (or REF=...)")
    out = {"hist_logregression": extract_logreg(os.path.join(ref, "tests/py/test_hist_logregression.py")),
           "sklearn_classification": extract_sklearn(os.path.join(ref, "tests/py/test_sklearn_classification.py")),
           "config": {"objective": 1, "method": 1,
                      "internals": {"double_precision": True, "compute_overlap": 2,
                                    "use_hist_subtraction_trick": True, "upload_features": True,
                                    "hist_size": 255},
                      "verbose": {"gpu": False, "booster": False, "data": False},
                      "tree": {"eta": 0.2, "max_depth": None, "gamma": 0.0, "min_child_weight": 2.0,
                               "min_leaf_size": 0, "colsample_bytree": 1.0, "colsample_bylevel": 1.0,
                               "lambda": 0.0, "alpha": 0.0}}}
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "iris_hist_golden.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=0, separators=(",", ":"))
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
