"""Graph containers with the reference's field names (jittor_geometric/data/data.py:42-52).

``CSR`` rows are keyed by edge source, ``CSC`` columns by edge destination; both
hold int32 index tensors and fp32 weights on a CUDA device.
"""


class CSR:
    def __init__(self, column_indices=None, row_offset=None, edge_weight=None):
        self.column_indices = column_indices
        self.row_offset = row_offset
        self.edge_weight = edge_weight


class CSC:
    def __init__(self, row_indices=None, column_offset=None, edge_weight=None):
        self.row_indices = row_indices
        self.column_offset = column_offset
        self.edge_weight = edge_weight
