"""Backend selector: deepnet/choose_matrix_library.py:1-16 with a third branch.

USE_GPU=b200 selects this library (`cm` = deepnet_b200.b200mat); `yes`/`auto`/`no`
keep the reference's meaning (cudamat / eigenmat, which must be importable).
"""
import os

use_gpu = os.environ.get("USE_GPU", "b200")
assert use_gpu in ["auto", "yes", "no", "b200"], "environment variable USE_GPU, should be one of 'auto', 'yes', 'no', 'b200'."

if use_gpu == "b200":
    from deepnet_b200 import b200mat as cm
elif use_gpu in ("auto", "yes"):
    try:
        import cudamat as cm
        from cudamat import cudamat_conv as cc  # noqa: F401
        from cudamat import gpu_lock  # noqa: F401
    except Exception:
        if use_gpu == "yes":
            raise
        print("Failed to import cudamat. Using eigenmat. No GPU will be used.")
        import eigenmat as cm
else:
    import eigenmat as cm
