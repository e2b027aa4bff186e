"""Checker-side restatement of how the reference's Python driver reads a per-layer program's
standard output (PefCounterForOperator, evalution/conv2d_timing.py:37-81): which lines it picks
and how it cuts the numbers out of them.  Used to check that the engine's `spconv2d_test`
programs keep that driver working."""


def parse_operator_output(lines):
    """(op_config dict of strings, time in ms, FLOPS figure, lines the driver would log).

    As the driver does: a line containing "FLOPS of" is split at " :" and loses its last
    character ("T"); a line containing "Time of" is split at " :" and loses its last two ("ms"),
    the word before " :" naming the vendor; "[Config] k = v, k = v, ..." fills the config; lines
    containing "Pass" or "best tile size" are logged; a line containing "Error" raises when the
    vendor is "Sparse".
    """
    op_config, vendor_time, vendor_flops, vendor, logged = {}, -1.0, -1.0, None, []
    for line in lines:
        line = line.strip()
        if "FLOPS of" in line:
            _, flops = line.split(" :")
            vendor_flops = float(flops[:-1])
        if "Time of" in line:
            key, t = line.split(" :")
            vendor = key.split(" ")[-1]
            vendor_time = float(t[:-2])
        if "[Config]" in line:
            _, config = line.split("[Config] ")
            for item in config.split(", "):
                k, v = item.split(" = ")
                op_config[k] = v
        if "Pass" in line:
            logged.append(line)
        if "Error" in line:
            if vendor != "Sparse":
                continue
            raise ValueError(line)
        if "best tile size" in line:
            logged.append(line)
    return op_config, vendor_time, vendor_flops, logged
