"""Stand-in so that ``from max.dtype import DType`` in the reference's test helpers gives the
dtype enum of the package under test."""
