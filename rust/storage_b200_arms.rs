// COMPILE-UNVERIFIED.  The arms to add to crates/weta-tensor/src/storage.rs so that `Storage` dispatches to the
// B200 backend next to the existing `Cuda` variant (storage.rs:11-15, 83-119).  With the `b200` Cargo feature:
//
//   [dependencies] weta-b200 = { workspace = true, optional = true }     [features] b200 = ["dep:weta-b200"]

pub enum Storage {
    Cpu(CpuStorage),
    #[cfg(feature = "cuda")]
    Cuda(weta_cuda::CudaStorage),
    #[cfg(feature = "b200")]
    B200(weta_b200::B200Storage),
}

// inside dispatch1! (storage.rs:83-99), after the Cuda arm:
//
//     #[cfg(feature = "b200")]
//     Storage::B200(s) => {
//         let $b = weta_b200::backend(s.ordinal()).expect("B200 device");
//         let $x = v!(s, $l, $dt);
//         Storage::B200($body)
//     }
//
// inside dispatch2! (storage.rs:101-119), after the (Cuda, Cuda) arm:
//
//     #[cfg(feature = "b200")]
//     (Storage::B200(a), Storage::B200(c)) => {
//         let $b = weta_b200::backend(a.ordinal()).expect("B200 device");
//         let ($x, $y) = (v!(a, $la, $dt), v!(c, $lb, $dt));
//         Storage::B200($body)
//     }
//
// and wherever storage.rs asks the GPU crate about the machine (storage.rs:44, 57, 68):
//
//     pub fn cuda_is_available() -> bool { #[cfg(feature = "b200")] { weta_b200::is_available() } ... }
//     pub fn cuda_profile_report() -> Option<String> { #[cfg(feature = "b200")] { weta_b200::profile_report() } ... }
//     pub fn cuda_device_count() -> usize { #[cfg(feature = "b200")] { weta_b200::device_count() } ... }
//
// `Device::Cuda(i)` keeps naming the GPU (crates/weta-core/src/lib.rs:37); which GPU crate serves it is the
// feature's choice, so weta-autograd, weta-nn and weta-optim compile unchanged.
