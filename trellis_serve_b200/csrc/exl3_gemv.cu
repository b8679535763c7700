// Host side of the decode GEMV: work split, shared-memory budget, dispatch on K.
#include "exl3_gemv_kernel.cuh"

namespace exl3 {

static int g_mode_override = -1;
[[maybe_unused]] static int g_tl_next_slot = 0;

#ifdef EXL3_TIMELINE
__device__ unsigned long long g_timeline[TL_SLOTS][TL_CTAS][TL_POINTS];
static unsigned long long* g_tl_base = nullptr;
extern "C" int exl3_debug_timeline(unsigned long long* host_out, int* next_slot)
{
    if (next_slot) *next_slot = g_tl_next_slot;
    return (int)cudaMemcpyFromSymbol(host_out, g_timeline, sizeof(g_timeline));
}
extern "C" void exl3_debug_timeline_reset(void) { g_tl_next_slot = 0; }
#endif


int gemv_default_mode(int codebook)
{
    if (codebook_family(codebook) == FAM_MUL1) return GEMV_PAIRED;
    return g_mode_override >= 0 ? g_mode_override : GEMV_SPLIT;
}

void gemv_set_mode_override(int mode) { g_mode_override = mode; }

constexpr size_t GEMV_FIXED_SMEM = 256 + GEMV_MAX_ROWS * 128 * 4;
constexpr size_t GEMV_RING_TARGET = 96 * 1024;
constexpr size_t GEMV_STAGE_TARGET = 32 * 1024;

WorkspaceLayout workspace_layout(int rows, int k, int n_total, int n_shards)
{
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const int r = rows < GEMV_MAX_ROWS ? (rows < 1 ? 1 : rows) : GEMV_MAX_ROWS;
    WorkspaceLayout w;
    w.err_off = 0;
    w.counters_off = WS_HEADER_BYTES;
    w.xf_off = WS_SCRATCH_OFF;
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

// Work split and shared-memory plan of one launch.  With `fused` the fragment slots of the in-kernel rotation are
// budgeted first and the ring takes what is left; an error status when that leaves fewer than two stages.
static int plan_gemv(const GemvArgs& a, const DeviceInfo* d, bool fused, GemvLaunch& l, size_t& smem)
{
    l.a = a;
    l.tl = nullptr;
    l.KG = a.k / 128;
    l.NB = a.n_total / 128;
    const long long units = (long long)l.KG * l.NB;
    int grid = d->sm_count * GEMV_CTAS_PER_SM;
    if (grid > GEMV_MAX_GRID) grid = GEMV_MAX_GRID;
    if (units < grid) grid = (int)units;
    l.grid = grid;
    l.units_q = (int)(units / grid);
    l.units_r = (int)(units % grid);
    const int fw = gemv_frag_words(a.mode);
    // Stage = as many whole units as make one bulk copy of 32 KB or a little more; two or three stages in flight.  When the
    // fragment slots of the in-kernel rotation leave no room for two such stages, smaller stages are tried.
    const uint32_t unit_bytes = 2048u * a.K;
    const long long per_cta = units / grid;
    const long long per_cta_max = per_cta + (l.units_r ? 1 : 0);
    size_t xs_bytes = 0;
    if (fused) xs_bytes = GEMV_XS_ZERO_BYTES + (size_t)(l.units_q + 1) * gemv_xs_slot_bytes(a.mode, a.rows);
    const size_t budget = (size_t)d->max_smem_optin / GEMV_CTAS_PER_SM - 2048 - GEMV_FIXED_SMEM;
    // Without the in-kernel rotation the fragments of a stage's units are copied behind its weights (see the kernel).
    const uint32_t frag_bytes = fused ? 0u : gemv_xs_slot_bytes(a.mode, a.rows);
    int stages = 0;
    for (size_t target = GEMV_STAGE_TARGET; target >= 8 * 1024 && stages < 2; target -= 8 * 1024) {
        int ups = (int)((target + unit_bytes - 1) / unit_bytes);
        // Short ranges travel as one copy: the copies of a launch start while the kernel ahead of it is still finishing,
        // so nothing is gained by cutting a small range into several copies, each of which pays the copy engine's fixed cost.
        if (per_cta_max < ups) ups = (int)per_cta_max;
        if (ups < 1) ups = 1;
        l.units_per_stage = ups;
        l.stage_stride = (uint32_t)ups * (unit_bytes + frag_bytes);
        if (xs_bytes + 2 * (size_t)l.stage_stride > budget) continue;
        stages = (int)(GEMV_RING_TARGET / l.stage_stride);
        const int cap = (int)((budget - xs_bytes) / l.stage_stride);
        if (stages > cap) stages = cap;
        if (stages > GEMV_MAX_STAGES) stages = GEMV_MAX_STAGES;
    }
    if (stages < 2) return EXL3_ERR_UNSUPPORTED_ROWS;
    l.stages = stages;
    l.xs_off = (uint32_t)(GEMV_FIXED_SMEM + (size_t)stages * l.stage_stride);
    smem = l.xs_off + xs_bytes;
    const CodebookConst c = codebook_const(a.codebook);
    l.mul = c.mul;
    l.add = c.add;
    l.xf_shard_stride = (long long)(a.k / 16) * a.rows * 4 * fw;
    l.pw = make_pow2();
    l.zeros = reinterpret_cast<const unsigned char*>(a.err) + 64;      // the workspace header stays zero past the error word
    return EXL3_OK;
}

bool gemv_rotates_input(const GemvArgs& a)
{
    const DeviceInfo* d = current_device_info();
    if (!d || (a.x ? !a.suh : !a.xf_staged) || a.rotated || a.rows < 1 || a.rows > GEMV_FUSED_ROWS) return false;
    if (a.k < 128 || a.n_total < 128) return false;
    GemvLaunch l;
    size_t smem;
    return plan_gemv(a, d, true, l, smem) == EXL3_OK;
}

int launch_gemv(const GemvArgs& a, cudaStream_t st)
{
    const DeviceInfo* d = current_device_info();
    if (!d) return EXL3_ERR_NOT_INITIALISED;
    if (a.rows < 1 || a.rows > GEMV_MAX_ROWS) return EXL3_ERR_UNSUPPORTED_ROWS;
    const long long units = (long long)(a.k / 128) * (a.n_total / 128);
    if (units == 0) return EXL3_OK;
    if (units >= (1ll << 31)) return EXL3_ERR_BAD_SHAPE;
    GemvLaunch l;
    size_t smem = 0;
    if (int rc = plan_gemv(a, d, a.x != nullptr || a.xf_staged, l, smem)) return rc;
#ifdef EXL3_TIMELINE
    if (!g_tl_base) cudaGetSymbolAddress(reinterpret_cast<void**>(&g_tl_base), g_timeline);
    l.tl = g_tl_base + (size_t)(g_tl_next_slot++ % TL_SLOTS) * TL_CTAS * TL_POINTS;
#endif
    switch (a.K) {
        case 2: return launch_gemv_for_k<2>(l, smem, st);
        case 3: return launch_gemv_for_k<3>(l, smem, st);
        case 4: return launch_gemv_for_k<4>(l, smem, st);
        case 5: return launch_gemv_for_k<5>(l, smem, st);
        case 6: return launch_gemv_for_k<6>(l, smem, st);
        case 7: return launch_gemv_for_k<7>(l, smem, st);
        case 8: return launch_gemv_for_k<8>(l, smem, st);
    }
    return EXL3_ERR_UNSUPPORTED_K;
}

}  // namespace exl3
