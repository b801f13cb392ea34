"""In-process stand-in for an etcd v2 server and the ``python-etcd`` client in front of it, for
tests of the rendezvous handler: one ``Server`` holds the key space (values, directories, TTLs,
modification indices), any number of ``Client`` objects talk to it from different threads.

Only what the rendezvous code uses is modelled: ``get``/``read``, ``write``/``set`` with
``prevExist`` / ``prevValue`` / ``ttl`` / ``dir``, ``update`` (compare on the modification index),
``test_and_set``, ``delete`` with ``prevValue``, ``watch`` with an index and a timeout, ``refresh``
and ``Lock``.  The module also plays the role of the ``etcd`` module itself (exception classes,
``Client``, ``Lock``), so it can be handed to code that expects ``import etcd``.
"""
import threading
import time


class EtcdException(Exception):
    pass


class EtcdKeyNotFound(EtcdException):
    pass


class EtcdAlreadyExist(EtcdException):
    pass


class EtcdCompareFailed(EtcdException):
    pass


class EtcdWatchTimedOut(EtcdException):
    pass


class EtcdEventIndexCleared(EtcdException):
    pass


class EtcdNotFile(EtcdException):
    pass


class EtcdResult:
    def __init__(self, key, value, modified_index, etcd_index, is_dir=False, ttl=None, children=()):
        self.key, self.value, self.dir, self.ttl = key, value, is_dir, ttl
        self.modifiedIndex = modified_index
        self.etcd_index = etcd_index
        self._children = list(children)

    @property
    def children(self):
        return iter(self._children)

    def __repr__(self):
        return f"EtcdResult({self.key!r}, {self.value!r}, idx={self.modifiedIndex})"


class _Node:
    __slots__ = ("value", "is_dir", "index", "expires")

    def __init__(self, value, is_dir, index, expires):
        self.value, self.is_dir, self.index, self.expires = value, is_dir, index, expires


class Server:
    def __init__(self):
        self.nodes = {}                 # full key -> _Node
        self.index = 0
        self.history = []               # (index, key) of every change
        self.cond = threading.Condition()

    # ---- helpers (caller holds self.cond)
    def _expire(self):
        now = time.time()
        dead = [k for k, n in self.nodes.items() if n.expires is not None and n.expires <= now]
        for k in dead:
            for kk in [x for x in self.nodes if x == k or x.startswith(k + "/")]:
                del self.nodes[kk]
            self.index += 1
            self.history.append((self.index, k))
        if dead:
            self.cond.notify_all()

    def _mkparents(self, key):
        parts = key.strip("/").split("/")
        for i in range(1, len(parts)):
            d = "/" + "/".join(parts[:i])
            if d not in self.nodes:
                self.nodes[d] = _Node(None, True, self.index, None)

    def _result(self, key):
        n = self.nodes[key]
        ttl = None if n.expires is None else max(int(n.expires - time.time()), 0)
        children = []
        if n.is_dir:
            depth = key.count("/") + 1
            for k, c in sorted(self.nodes.items()):
                if k.startswith(key + "/") and k.count("/") == depth:
                    cttl = None if c.expires is None else max(int(c.expires - time.time()), 0)
                    children.append(EtcdResult(k, c.value, c.index, self.index, c.is_dir, cttl))
        return EtcdResult(key, n.value, n.index, self.index, n.is_dir, ttl, children)

    def dump(self):
        """{key: value} of every file node (directories omitted), for traces."""
        with self.cond:
            self._expire()
            return {k: n.value for k, n in sorted(self.nodes.items()) if not n.is_dir}


def _norm(key):
    key = "/" + key.strip("/")
    while "//" in key:
        key = key.replace("//", "/")
    return key


class Client:
    def __init__(self, server=None, **_ignored):
        self.server = server if server is not None else Server()
        self.machines = ["fake://in-process"]

    # ------------------------------------------------------------------ reads
    def get(self, key, **kw):
        return self.read(key, **kw)

    def read(self, key, wait=False, waitIndex=None, timeout=None, recursive=False, **_):
        if wait:
            return self.watch(key, index=waitIndex, timeout=timeout, recursive=recursive)
        key = _norm(key)
        s = self.server
        with s.cond:
            s._expire()
            if key not in s.nodes:
                raise EtcdKeyNotFound(f"Key not found : {key}")
            return s._result(key)

    # ------------------------------------------------------------------ writes
    def write(self, key, value, ttl=None, dir=False, append=False, prevExist=None, prevValue=None, prevIndex=None, **_):
        key = _norm(key)
        s = self.server
        with s.cond:
            s._expire()
            exists = key in s.nodes
            if prevExist is False and exists:
                raise EtcdAlreadyExist(f"Key already exists : {key}")
            if prevExist is True and not exists:
                raise EtcdKeyNotFound(f"Key not found : {key}")
            if prevValue is not None:
                if not exists:
                    raise EtcdKeyNotFound(f"Key not found : {key}")
                if s.nodes[key].value != prevValue:
                    raise EtcdCompareFailed(f"Compare failed : [{prevValue} != {s.nodes[key].value}]")
            if prevIndex is not None:
                if not exists:
                    raise EtcdKeyNotFound(f"Key not found : {key}")
                if s.nodes[key].index != prevIndex:
                    raise EtcdCompareFailed(f"Compare failed : [{prevIndex} != {s.nodes[key].index}]")
            if exists and s.nodes[key].is_dir and not dir:
                raise EtcdNotFile(f"Not a file : {key}")
            s._mkparents(key)
            s.index += 1
            expires = None if ttl is None else time.time() + ttl
            s.nodes[key] = _Node(None if dir else (value if value is None else str(value)), bool(dir), s.index, expires)
            s.history.append((s.index, key))
            s.cond.notify_all()
            return s._result(key)

    def set(self, key, value, ttl=None):
        return self.write(key, value, ttl=ttl)

    def update(self, obj):
        """Write back a result that was read before: compare on its modification index."""
        return self.write(obj.key, obj.value, ttl=obj.ttl, prevIndex=obj.modifiedIndex)

    def test_and_set(self, key, value, prev_value, ttl=None):
        return self.write(key, value, prevValue=prev_value, ttl=ttl)

    def refresh(self, key, ttl, **_):
        key = _norm(key)
        s = self.server
        with s.cond:
            s._expire()
            if key not in s.nodes:
                raise EtcdKeyNotFound(f"Key not found : {key}")
            s.nodes[key].expires = time.time() + ttl
            return s._result(key)

    def delete(self, key, recursive=None, dir=None, prevValue=None, prevIndex=None, **_):
        key = _norm(key)
        s = self.server
        with s.cond:
            s._expire()
            if key not in s.nodes:
                raise EtcdKeyNotFound(f"Key not found : {key}")
            if prevValue is not None and s.nodes[key].value != prevValue:
                raise EtcdCompareFailed(f"Compare failed : [{prevValue} != {s.nodes[key].value}]")
            if prevIndex is not None and s.nodes[key].index != prevIndex:
                raise EtcdCompareFailed("Compare failed")
            res = s._result(key)
            for kk in [x for x in s.nodes if x == key or x.startswith(key + "/")]:
                del s.nodes[kk]
            s.index += 1
            s.history.append((s.index, key))
            s.cond.notify_all()
            return res

    # ------------------------------------------------------------------ watch
    def watch(self, key, index=None, timeout=None, recursive=None):
        key = _norm(key)
        s = self.server
        deadline = None if timeout is None or timeout == 0 else time.time() + timeout
        with s.cond:
            while True:
                s._expire()
                start = index if index is not None else s.index + 1
                for idx, k in s.history:
                    if idx >= start and (k == key or (recursive and k.startswith(key + "/"))):
                        if k in s.nodes:
                            return s._result(k)
                        return EtcdResult(k, None, idx, s.index)
                if index is None:
                    index = s.index + 1
                remaining = None if deadline is None else deadline - time.time()
                if remaining is not None and remaining <= 0:
                    raise EtcdWatchTimedOut(f"Watch timed out : {key}")
                # wake up regularly: TTL expiry is only noticed when somebody looks
                s.cond.wait(0.05 if remaining is None else min(0.05, remaining))


class Lock:
    """python-etcd's ``Lock(client, name)``: acquire(blocking, lock_ttl) / release()."""

    _locks = {}
    _guard = threading.Lock()

    def __init__(self, client, lock_name):
        with Lock._guard:
            # a client that is a proxy of a server in another process has no `server`: the lock is
            # then local to this process
            self._lock = Lock._locks.setdefault((id(getattr(client, "server", client)), lock_name), threading.Lock())
        self.is_taken = False

    def acquire(self, blocking=True, lock_ttl=3600, timeout=0):
        self.is_taken = self._lock.acquire(blocking)
        return self.is_taken

    def release(self):
        if self.is_taken:
            self._lock.release()
            self.is_taken = False
        return True


# ---------------------------------------------------------------------------------- across processes
# One key space for several worker processes: a manager process holds the Server, workers get
# proxies of a Client in front of it (results and exceptions travel by pickle).
from multiprocessing.managers import BaseManager  # noqa: E402

_SHARED = None


def _shared_client():
    global _SHARED
    if _SHARED is None:
        _SHARED = Server()
    return Client(_SHARED)


class EtcdManager(BaseManager):
    pass


EtcdManager.register("Client", callable=_shared_client,
                     exposed=("get", "read", "write", "set", "update", "test_and_set", "refresh", "delete", "watch"))


def start_shared_server(authkey=b"fake-etcd"):
    """Starts the manager process; returns (manager, address).  Workers call ``connect(address)``."""
    import multiprocessing as mp
    mgr = EtcdManager(address=("127.0.0.1", 0), authkey=authkey, ctx=mp.get_context("spawn"))
    mgr.start()
    return mgr, mgr.address


def connect(address, authkey=b"fake-etcd"):
    mgr = EtcdManager(address=tuple(address), authkey=authkey)
    mgr.connect()
    return mgr.Client()
