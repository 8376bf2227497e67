"""Where the built library lives (shared by the build recipe and the loader)."""
import os

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
# PLX_SM100_LIBRARY points the loader at a libplx_sm100.so built elsewhere (same C ABI version)
LIB_PATH = os.environ.get("PLX_SM100_LIBRARY") or os.path.join(LIB_DIR, "libplx_sm100.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
