"""Error types.  The reference has one enum, ``XrtError`` (crates/xrt-core/src/lib.rs:203-227);
here each family that a caller may want to catch on its own is a subclass of it."""


class XrtError(Exception):
    """Base of every error the library raises on purpose."""


class ConfigError(XrtError):
    """config.json is missing a key, holds a contradictory value, or names an unknown architecture
    (``InvalidMetadata`` in the reference)."""


class Unsupported(XrtError):
    """A valid request that this library does not implement (``Unsupported`` in the reference)."""


class WeightError(XrtError):
    """Tensors of a model file do not fit the model: missing, unexpected, wrong shape or dtype
    (``InvalidTensor`` in the reference)."""


class CacheError(XrtError):
    """Misuse or exhaustion of the cache: no free slot or block, a slot freed twice, a step that
    does not continue where the slot stands."""


class KernelError(XrtError):
    """The CUDA extension is missing, cannot be built, or refuses the sizes it was given."""


class RuntimeFault(XrtError):
    """A request the engine cannot run as asked: empty prompt, token id outside the vocabulary,
    prompt longer than the context (``Runtime`` / ``Model`` in the reference)."""
