"""Plays the part of IREE's executable-plugin loader for the tests: ctypes mirrors of the v0
plugin interface (runtime/src/iree/hal/local/executable_plugin.h:154-175 header, :186-189 query,
:386-461 environment, resolve parameters and the plugin struct) and a tiny host allocator."""
import ctypes as C
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN_PATH = os.path.join(ROOT, "iree_b200", "libiree_uk_b200_plugin.so")

VERSION_0_1 = 1
STATUS_OK, STATUS_INVALID_ARGUMENT, STATUS_NOT_FOUND = 0, 3, 5
RESOLUTION_MISSING_OPTIONAL = 1


class Header(C.Structure):
    _fields_ = [("version", C.c_uint32), ("name", C.c_char_p), ("description", C.c_char_p),
                ("features", C.c_uint32), ("sanitizer", C.c_int32), ("reserved", C.c_uint64 * 8)]


ALLOC_CTL = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_void_p))


class Allocator(C.Structure):
    _fields_ = [("self", C.c_void_p), ("ctl", ALLOC_CTL)]


class Environment(C.Structure):
    _fields_ = [("host_allocator", Allocator)]


class StringView(C.Structure):
    _fields_ = [("data", C.c_char_p), ("size", C.c_size_t)]


class StringPair(C.Structure):
    _fields_ = [("key", StringView), ("value", StringView)]


class ResolveParams(C.Structure):
    _fields_ = [("count", C.c_size_t), ("symbol_names", C.POINTER(C.c_char_p)),
                ("out_fn_ptrs", C.POINTER(C.c_void_p)), ("out_fn_contexts", C.POINTER(C.c_void_p))]


LOAD_FN = C.CFUNCTYPE(C.c_void_p, C.POINTER(Environment), C.c_size_t, C.POINTER(StringPair),
                      C.POINTER(C.c_void_p))
UNLOAD_FN = C.CFUNCTYPE(None, C.c_void_p)
RESOLVE_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.POINTER(ResolveParams), C.POINTER(C.c_uint32))
IMPORT_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p)


class PluginV0(C.Structure):
    _fields_ = [("header", C.POINTER(Header)), ("load", LOAD_FN), ("unload", UNLOAD_FN),
                ("resolve", RESOLVE_FN)]


def available():
    return os.path.exists(PLUGIN_PATH)


class Loader:
    """query -> load -> resolve -> (calls) -> unload, as the runtime does it."""

    def __init__(self, params=()):
        self.lib = C.CDLL(PLUGIN_PATH)
        self.lib.iree_hal_executable_plugin_query.restype = C.POINTER(PluginV0)
        self.lib.iree_hal_executable_plugin_query.argtypes = [C.c_uint32, C.c_void_p]
        self.lib.iree_uk_b200_plugin_configure.restype = C.c_int
        self.lib.iree_uk_b200_plugin_configure.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p,
                                                           C.c_size_t]
        self.lib.iree_uk_b200_plugin_last_status.restype = C.c_int
        self.lib.iree_uk_b200_plugin_last_status.argtypes = [C.c_void_p]
        self.live = {}  # allocations handed out, so that leaks and double frees show

        libc = C.CDLL(None)
        libc.malloc.restype, libc.malloc.argtypes = C.c_void_p, [C.c_size_t]
        libc.free.argtypes = [C.c_void_p]

        def ctl(_self, command, cmd_params, inout_ptr):
            if command in (0, 1):  # malloc / calloc: params -> {byte_length}
                n = C.cast(cmd_params, C.POINTER(C.c_size_t))[0]
                p = libc.malloc(max(n, 1))
                if command == 1:
                    C.memset(p, 0, n)
                self.live[p] = n
                inout_ptr[0] = p
                return STATUS_OK
            if command == 3:  # free
                p = inout_ptr[0]
                assert p in self.live, "free of a pointer this allocator did not hand out"
                del self.live[p]
                libc.free(p)
                return STATUS_OK
            return 12  # UNIMPLEMENTED (realloc is not used by the plugin)

        self._ctl = ALLOC_CTL(ctl)
        self.env = Environment(Allocator(None, self._ctl))
        self.plugin = self.query(VERSION_0_1)
        self.self_ptr = C.c_void_p()
        pairs = (StringPair * max(len(params), 1))()
        self._keep = []
        for i, (k, v) in enumerate(params):
            kb, vb = k.encode(), v.encode()
            self._keep += [kb, vb]
            pairs[i] = StringPair(StringView(kb, len(kb)), StringView(vb, len(vb)))
        self.load_status = self.plugin.contents.load(C.byref(self.env), len(params), pairs,
                                                     C.byref(self.self_ptr)) or 0

    def query(self, max_version):
        return self.lib.iree_hal_executable_plugin_query(max_version, None)

    def resolve(self, names, preset=None):
        """Returns (status code, resolution bits, [function pointers], [contexts])."""
        n = len(names)
        arr = (C.c_char_p * n)(*[s.encode() for s in names])
        fns = (C.c_void_p * n)(*(preset or [None] * n))
        ctxs = (C.c_void_p * n)()
        rp = ResolveParams(n, arr, fns, ctxs)
        bits = C.c_uint32(0xFFFFFFFF)
        st = self.plugin.contents.resolve(self.self_ptr, C.byref(rp), C.byref(bits)) or 0
        return st & 0x1F, bits.value, list(fns), list(ctxs)

    def configure(self, stream, workspace=None, workspace_bytes=0):
        return self.lib.iree_uk_b200_plugin_configure(self.self_ptr, stream, workspace,
                                                      workspace_bytes)

    def last_status(self):
        return self.lib.iree_uk_b200_plugin_last_status(self.self_ptr)

    def unload(self):
        self.plugin.contents.unload(self.self_ptr)
        assert not self.live, "the plugin leaked host allocations"
