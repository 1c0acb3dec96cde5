"""TEST INFRASTRUCTURE: pure-Python restatement of the reference's host-side integer logic
around the attention op (small cases only). PARITY UNPINNED: the reference has no unit test
for these functions; they are restated from its source and checked on hand-derived cases.

  KVPoolRef            KVPool::ref / free_list, kv_alloc / kv_retain / kv_release
                       (src/model/impl/model.h:387-411, :722-737; set-up forest.h:59-61)
  target_blocks        Forest::target_blocks (src/model/impl/forest.h:1785-1811)
  target_new_blocks    src/model/impl/forest.h:1819-1829
  save_entries         add_saves (forest.h:2488-2499)
  row_table            kv_row_table (forest.h:1739-1749)
  tree_rows            leaf hosting (forest.h:2201-2220) + row records (forest.h:2374-2442)
"""


class KVFull(RuntimeError):
    pass


class KVPoolRef:
    def __init__(self, n_blocks: int, bt: int):
        self.bt = bt
        self.ref = [0] * n_blocks
        self.free_list = list(range(n_blocks - 1, -1, -1))

    def alloc(self) -> int:
        if not self.free_list:
            raise KVFull("KV cache full")
        b = self.free_list.pop()
        self.ref[b] = 1
        return b

    def retain(self, b: int):
        self.ref[b] += 1

    def release(self, b: int):
        self.ref[b] -= 1
        if self.ref[b] == 0:
            self.free_list.append(b)


def target_blocks(pool: KVPoolRef, parent_blocks, P, w0, end, in_place):
    bt = pool.bt
    out, cow = [], []
    keep = w0 // bt
    i = 0
    while i < keep and i < len(parent_blocks):
        out.append(parent_blocks[i])
        pool.retain(parent_blocks[i])
        i += 1
    need = (end + bt - 1) // bt
    for i in range(keep, need):
        has_parent = i < len(parent_blocks) and i * bt < P
        if has_parent and in_place and pool.ref[parent_blocks[i]] == 1:
            out.append(parent_blocks[i])
            pool.retain(parent_blocks[i])
            continue
        nb = pool.alloc()
        if has_parent:
            cow.append((parent_blocks[i], nb))
        out.append(nb)
    return out, cow


def target_new_blocks(pool: KVPoolRef, parent_blocks, P, w0, end, in_place):
    bt = pool.bt
    i = w0 // bt
    n = (end + bt - 1) // bt - i
    if n > 0 and in_place and parent_blocks is not None and i < len(parent_blocks) and i * bt < P and pool.ref[parent_blocks[i]] == 1:
        n -= 1
    return max(n, 0)


def save_entries(blocks, bt, P, base_row, n_rows):
    return [(base_row + i, blocks[(P + i) // bt], (P + i) % bt, 0) for i in range(n_rows)]


def row_table(entries, rows):
    t = [-1] * (max(rows, 1) * 4)
    for (src_row, block, pos, _pad) in entries:
        j = 0 if t[4 * src_row] < 0 else 2
        if j == 2 and t[4 * src_row + 2] >= 0:
            raise ValueError("a row saved into more than two slots")
        t[4 * src_row + j] = block
        t[4 * src_row + j + 1] = pos
    return t


def tree_rows(root, leaves, base, pnext, root_pos=None, noncausal=False, score_root=False):
    """Returns dict(host, off, tok, pos, desc, readouts, M, next_root); leaves = list of token lists."""
    Tr, NL = len(root), len(leaves)
    ln = [len(x) for x in leaves]
    host = [-1] * NL
    for i in range(NL):
        h = i
        for j in range(NL):
            if j == i or ln[j] < ln[i]:
                continue
            if ln[j] == ln[i] and j > i:
                continue
            if ln[j] < ln[h] or (ln[j] == ln[h] and j >= h):
                continue
            if leaves[j][:ln[i]] == leaves[i]:
                h = j
        host[i] = h
    off, leaf_rows = [0] * NL, 0
    for i in range(NL):
        if host[i] == i:
            off[i] = leaf_rows
            leaf_rows += ln[i]
    M = Tr + leaf_rows
    tok, pos, desc = [0] * M, [[0, 0, 0, 0] for _ in range(M)], [[0, 0, 0, 0] for _ in range(M)]
    pmax = pnext - 1
    for j in range(Tr):
        pt = ph = pw = pnext + j
        if root_pos is not None:
            pt, ph, pw = root_pos[j]
        tok[j] = root[j]
        pos[j] = [pt, ph, pw, 0]
        pmax = max(pmax, pt, ph, pw)
        desc[j] = [0, 0, Tr if noncausal else 0, 0]
    next_root = pmax + 1
    readouts = []
    for i in range(NL):
        h = host[i]
        start = Tr + off[h]
        readouts.append(base + start + ln[i] - 1)
        if h != i:
            continue
        for j in range(ln[i]):
            r = start + j
            tok[r] = leaves[i][j]
            pos[r] = [next_root + j] * 3 + [0]
            desc[r] = [start, 0, Tr, 0]
    if score_root or NL == 0:
        readouts.append(base + Tr - 1)
    return dict(host=host, off=off, tok=tok, pos=pos, desc=desc, readouts=readouts, M=M, next_root=next_root)


def anc_masks(parents):
    masks = []
    for i, p in enumerate(parents):
        masks.append((1 << i) | (masks[p] if p >= 0 else 0))
    return masks
