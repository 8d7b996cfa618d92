"""A plain Python builder of a step's index arrays, for tests: the product fills them natively
(``nvh_prepare_step``); a CPU test holds the two to each other, and tests of single parts use this one to make
batches by hand, with block tables of their own choosing."""
import numpy as np

from nano_vllm_cpp_b200.engine.batch import BatchStager, StepBatch, batch_from_buffer, batch_layout


def build_batch(entries: list, infos: list, tables, max_blocks: int, device, stager=None,
                static_dev=None, table_filler=None, num_groups=None) -> StepBatch:
    """``infos``: EntryInfo per entry; ``tables``: per group, per entry, the list of page ids — or None with
    ``table_filler(group, entry, dst)``, which writes an entry's block table into an int32 array view.
    The block tables are written whole, [S, max_blocks] per group behind the other arrays (the product sends only
    the tables that changed and keeps the rest on the device).  With ``static_dev`` the arrays are written into that
    device buffer (at least as long) instead of a fresh one."""
    S = len(entries)
    T = sum(len(e.tokens) for e in entries)
    n_want = sum(len(e.want) for e in entries)
    G = len(tables) if tables is not None else num_groups
    seg, fixed = batch_layout(S, T, n_want, G, max_blocks, table_rows=[0] * G)    # no tables travel: dense ones follow
    total = fixed + G * S * max_blocks
    host = np.full(total, -1, dtype=np.int32)

    def put(name, values):
        o, n = seg[name]
        host[o:o + n] = values

    ids, pos, row_entry, cu, want = [], [], [], [0], []
    for i, (e, info) in enumerate(zip(entries, infos)):
        n = len(e.tokens)
        ids.extend(e.tokens)
        pos.extend(range(info.pos0, info.pos0 + n))
        row_entry.extend([i] * n)
        for w in e.want:
            if not (0 <= w < n):
                raise ValueError(f"request {e.rid!r}: wanted place {w} is not among its {n} tokens")
            want.append(info.row0 + w)
        cu.append(cu[-1] + n)
    put("ids", ids), put("pos", pos), put("row_entry", row_entry), put("cu", cu)
    put("pos0", [i.pos0 for i in infos]), put("slot", [i.slot for i in infos]), put("want", want)
    single = [i.row0 for i in infos if i.length == 1]
    put("single", single + [-1] * (S - len(single)))
    for g in range(G):
        o = fixed + g * S * max_blocks
        if tables is None:
            for i in range(S):
                if table_filler(g, i, host[o + i * max_blocks:o + (i + 1) * max_blocks]) > max_blocks:
                    raise ValueError("a request holds more pages than the block table is wide")
            continue
        for i, table in enumerate(tables[g]):
            if len(table) > max_blocks:
                raise ValueError("a request holds more pages than the block table is wide")
            host[o + i * max_blocks:o + i * max_blocks + len(table)] = table
    if stager is None:
        stager = BatchStager(device, depth=1)
    dev = stager.stage(host, static_dev)

    dense = [dev[fixed + g * S * max_blocks:fixed + (g + 1) * S * max_blocks].view(S, max_blocks) for g in range(G)]
    batch = batch_from_buffer(dev, seg, infos, S, T, G, max_blocks, int(host.nbytes), dense)
    batch.table_updates = None              # the tables above are complete: nothing is to be taken in
    return batch
