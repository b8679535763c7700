// Host side of the decode GEMV: work split, shared-memory budget, dispatch on K.
#include "exl3_gemv_kernel.cuh"

namespace exl3 {

static int g_mode_override = -1;

int gemv_default_mode(int codebook)
{
    if (codebook_family(codebook) == FAM_MUL1) return GEMV_PAIRED;
    return g_mode_override >= 0 ? g_mode_override : GEMV_SPLIT;
}

void gemv_set_mode_override(int mode) { g_mode_override = mode; }

constexpr size_t GEMV_FIXED_SMEM = 256 + GEMV_MAX_ROWS * 128 * 4;
constexpr size_t GEMV_RING_TARGET = 96 * 1024;

size_t gemv_smem_bytes(const GemvLaunch& l) { return GEMV_FIXED_SMEM + (size_t)l.stages * l.stage_stride; }

WorkspaceLayout workspace_layout(int rows, int k, int n_total, int n_shards)
{
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const int r = rows < GEMV_MAX_ROWS ? (rows < 1 ? 1 : rows) : GEMV_MAX_ROWS;
    WorkspaceLayout w;
    w.err_off = 0;
    w.counters_off = 256;
    w.xf_off = up(w.counters_off + (size_t)(n_total / 128) * sizeof(int));
    w.partials_off = up(w.xf_off + (size_t)n_shards * (k / 16) * r * 4 * 4 * sizeof(uint32_t));
    w.total = up(w.partials_off + (size_t)(GEMV_MAX_GRID + n_total / 128) * r * 128 * sizeof(float));
    return w;
}

int gemv_init_device()
{
    const DeviceInfo* d = current_device_info();
    if (!d) return EXL3_ERR_NOT_INITIALISED;
    int rc = EXL3_OK;
    if (rc == EXL3_OK) rc = gemv_set_attributes_for_k<2>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = gemv_set_attributes_for_k<3>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = gemv_set_attributes_for_k<4>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = gemv_set_attributes_for_k<5>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = gemv_set_attributes_for_k<6>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = gemv_set_attributes_for_k<7>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = gemv_set_attributes_for_k<8>(d->max_smem_optin);
    return rc;
}

int launch_gemv(const GemvArgs& a, cudaStream_t st)
{
    const DeviceInfo* d = current_device_info();
    if (!d) return EXL3_ERR_NOT_INITIALISED;
    if (a.rows < 1 || a.rows > GEMV_MAX_ROWS) return EXL3_ERR_UNSUPPORTED_ROWS;
    GemvLaunch l;
    l.a = a;
    l.KG = a.k / 128;
    l.NB = a.n_total / 128;
    const long long units = (long long)l.KG * l.NB;
    if (units == 0) return EXL3_OK;
    int grid = d->sm_count < GEMV_MAX_GRID ? d->sm_count : GEMV_MAX_GRID;
    if (units < grid) grid = (int)units;
    l.grid = grid;
    l.units_q = (int)(units / grid);
    l.units_r = (int)(units % grid);
    const int fw = gemv_frag_words(a.mode);
    l.xf_bytes = (uint32_t)(128 * fw * a.rows);
    l.stage_stride = (uint32_t)((2048u * a.K + l.xf_bytes + 127u) & ~127u);
    int stages = (int)(GEMV_RING_TARGET / l.stage_stride);
    const int cap = (int)((d->max_smem_optin - GEMV_FIXED_SMEM) / l.stage_stride);
    if (stages > cap) stages = cap;
    if (stages > GEMV_MAX_STAGES) stages = GEMV_MAX_STAGES;
    if (stages < 2) return EXL3_ERR_UNSUPPORTED_ROWS;
    l.stages = stages;
    const CodebookConst c = codebook_const(a.codebook);
    l.mul = c.mul;
    l.add = c.add;
    l.xf_shard_stride = (long long)(a.k / 16) * a.rows * 4 * fw;
    switch (a.K) {
        case 2: return launch_gemv_for_k<2>(l, st);
        case 3: return launch_gemv_for_k<3>(l, st);
        case 4: return launch_gemv_for_k<4>(l, st);
        case 5: return launch_gemv_for_k<5>(l, st);
        case 6: return launch_gemv_for_k<6>(l, st);
        case 7: return launch_gemv_for_k<7>(l, st);
        case 8: return launch_gemv_for_k<8>(l, st);
    }
    return EXL3_ERR_UNSUPPORTED_K;
}

}  // namespace exl3
