"""Small host helpers with the reference's names (sparse_dok/util.py:72-137, 289-293)."""
import torch


def next_prime(n):
    """Smallest prime larger than n (the reference uses sympy.nextprime for its hash parameters,
    cuda_closed_hashmap.py:76, 88)."""
    import sympy
    return int(sympy.nextprime(int(n)))


_STR2DTYPE = {
    "bool": torch.bool, "uint8": torch.uint8, "char": torch.uint8, "int8": torch.int8, "byte": torch.int8,
    "int16": torch.int16, "short": torch.int16, "int32": torch.int32, "int": torch.int32,
    "int64": torch.int64, "long": torch.int64, "float16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "float32": torch.float32, "float": torch.float32,
    "float64": torch.float64, "double": torch.float64,
}


def str2dtype(s):
    if isinstance(s, torch.dtype):
        return s
    if isinstance(s, str):
        if s not in _STR2DTYPE:
            raise ValueError(f"unrecognized type string {s}")
        return _STR2DTYPE[s]
    raise RuntimeError


_DTYPE2CTYPE = {
    torch.bool: "bool", torch.uint8: "uint8_t", torch.int8: "int8_t", torch.int16: "int16_t",
    torch.int32: "int32_t", torch.int64: "int64_t", torch.float16: "half", torch.bfloat16: "bfloat16",
    torch.float32: "float", torch.float64: "double",
}


def dtype2ctype(dtype):
    return _DTYPE2CTYPE.get(str2dtype(dtype))


def next_power_of_2(n):
    """n itself if it is a power of two, else the next one; 1 for n == 0 (sparse_dok/util.py:125-137)."""
    n = int(n)
    if n and not (n & (n - 1)):
        return n
    return 1 << n.bit_length()


def shape_to_stride(shape):
    """Row-major element strides of a contiguous tensor of `shape`."""
    out, acc = [], 1
    for s in reversed(tuple(shape)):
        out.append(acc)
        acc *= int(s)
    return tuple(reversed(out))


def consume_fresh_map_draws(n_buckets, key_size, n_new, rehash_factor=2.0, rehash_threshold=0.75):
    """Advances the global numpy random state by exactly what a never-used reference map of `n_buckets` consumes when
    its first `set` stores `n_new` distinct keys of `key_size` elements (cuda_closed_hashmap.py:66-113, 350-366): one
    draw per element for prime1, prime2, alpha1, alpha2, beta1, beta2, and the same again for the rebuilt table when
    the batch crosses the rehash threshold.  Used where this library skips an intermediate tensor that the reference
    builds, so that tensors created afterwards still get the parameters the reference would give them."""
    import numpy as np

    def draw(nb):
        prime1 = [next_prime(np.random.randint(nb, nb * 2)) for _ in range(key_size)]
        for _ in range(key_size):
            np.random.randint(0, 2 ** 60, dtype="int64")
        for _ in range(4):
            for p in prime1:
                np.random.randint(int(p))

    if n_new == 0:
        return
    draw(int(n_buckets))
    if n_new > int(rehash_threshold * n_buckets):
        draw(int(n_new * rehash_factor))
